// Host launchers of the f16/bf16 fused kernels: tensor maps, shape checks, launch.
#include "dense_ops.h"

#include <algorithm>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "gemm_fused.cuh"
#include "gemm_pair.cuh"
#include "gemm_pair_rs.cuh"
#include "ptx.cuh"

namespace cb {

static int encode_2d(const DriverApi *api, CUtensorMap *tm, CUtensorMapDataType dt, const void *base, uint64_t inner,
                     uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = api->TensorMapEncodeTiled(tm, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        const char *s = nullptr;
        api->GetErrorString(r, &s);
        set_error("cuTensorMapEncodeTiled failed: %s (base=%p inner=%llu outer=%llu stride=%llu box=%ux%u)",
                  s ? s : "?", base, (unsigned long long)inner, (unsigned long long)outer,
                  (unsigned long long)row_stride_bytes, box_inner, box_outer);
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

template <int OP, typename T, bool B_MN>
static int launch_kernel(const FusedParams &p, int grid, bool cooperative, cudaStream_t stream) {
    auto kern = fused_gemm_kernel<OP, T, B_MN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (e != cudaSuccess) {
        set_error("cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    if (cooperative) {
        // several emulated ranks wait on one another inside one launch: co-residency must be guaranteed
        void *args[] = {const_cast<FusedParams *>(&p)};
        e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(kern), dim3(grid), dim3(kGemmThreads), args,
                                        kGemmSmemBytes, stream);
    } else {
        kern<<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(p);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        set_error("kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

// CTA-pair (cta_group::2) kernels
template <typename K>
static int launch_pair_kernel(K kern, int threads, const FusedParams &p, int grid, bool cooperative, cudaStream_t stream,
                              int smem_bytes = kPairSmemBytes) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e == cudaSuccess) {
        if (cooperative) {
            void *args[] = {const_cast<FusedParams *>(&p)};
            e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(kern), dim3(grid), dim3(threads), args,
                                            smem_bytes, stream);
        } else {
            kern<<<grid, threads, smem_bytes, stream>>>(p);
            e = cudaGetLastError();
        }
    }
    if (e != cudaSuccess) {
        set_error("pair kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

template <typename K>
static int launch_pair_rs_kernel(K kern, const FusedParams &p, const RsMapsAll &maps, int grid, bool cooperative,
                                 cudaStream_t stream) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
    if (e == cudaSuccess) {
        if (cooperative) {
            void *args[] = {const_cast<FusedParams *>(&p), const_cast<RsMapsAll *>(&maps)};
            e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(kern), dim3(grid), dim3(kGemmThreads), args,
                                            kPairSmemBytes, stream);
        } else {
            kern<<<grid, kGemmThreads, kPairSmemBytes, stream>>>(p, maps);
            e = cudaGetLastError();
        }
    }
    if (e != cudaSuccess) {
        set_error("pair reduce-scatter kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

template <typename T, bool B_MN>
static int launch_pair(int op, const FusedParams &p, const RsMapsAll &maps, int grid, bool coop, cudaStream_t stream) {
    switch (op) {
        case OP_AGMM:
            // a single rank without a gather-result output moves nothing: the copy lanes' staging becomes a seventh stage
            if (p.world == 1 && !p.ranks[0].gather_out && !getenv("CATCCOS_AG_SIX_STAGES"))
                return launch_pair_kernel(pair_agmm_kernel<T, B_MN, kPStagesSolo>, kPairAgThreads, p, grid, coop, stream,
                                          kPairSoloSmemBytes);
            return launch_pair_kernel(pair_agmm_kernel<T, B_MN>, kPairAgThreads, p, grid, coop, stream);
        case OP_MMRS: return launch_pair_rs_kernel(pair_rs_kernel<OP_MMRS, T, B_MN>, p, maps, grid, coop, stream);
        case OP_MMA2A: return launch_pair_rs_kernel(pair_rs_kernel<OP_MMA2A, T, B_MN>, p, maps, grid, coop, stream);
        default: return launch_pair_rs_kernel(pair_rs_kernel<OP_MMAR, T, B_MN>, p, maps, grid, coop, stream);
    }
}

template <int OP, typename T>
static int launch_b(const FusedParams &p, int grid, bool coop, cudaStream_t s, bool b_mn) {
    return b_mn ? launch_kernel<OP, T, true>(p, grid, coop, s) : launch_kernel<OP, T, false>(p, grid, coop, s);
}
template <int OP>
static int launch_t(const FusedParams &p, int grid, bool coop, cudaStream_t s, bool bf16, bool b_mn) {
    return bf16 ? launch_b<OP, __nv_bfloat16>(p, grid, coop, s, b_mn) : launch_b<OP, __half>(p, grid, coop, s, b_mn);
}

int encode_rs_maps(const DriverApi *api, Team *t, RsMapsAll *maps, int op, CUtensorMapDataType dt,
                   void *const *outputs, int n_local, int m, int n, uint64_t symm_off, bool compute_only) {
    const int R = t->n_pes;
    const bool allreduce = op == OP_MMAR;
    const bool full_output = op == OP_MMAR || op == OP_MMA2A;      // the output holds all m rows; own rows at pe * mr
    const int mr = allreduce ? (m + R - 1) / R : m / R;
    auto rows_valid = [&](int d) { return std::min(m, (d + 1) * mr) - d * mr; };
    const size_t row_b = static_cast<size_t>(n) * 2;
    for (int l = 0; l < n_local; ++l) {
        const int pe = t->emulated ? l : t->my_pe;
        RsMaps &mp = maps->r[l];
        for (int d = 0; d < R; ++d) {
            const int rv_d = rows_valid(d), rv_me = rows_valid(pe);
            if (d == pe) {
                if (rv_me <= 0) continue;
                uint8_t *base = static_cast<uint8_t *>(outputs[l]) + (full_output ? static_cast<size_t>(pe) * mr * row_b : 0);
                int rc = encode_2d(api, &mp.out[d], dt, base, n, rv_me, row_b, 64, 32);
                if (rc) return rc;
                continue;
            }
            if (rv_d > 0) {
                // this rank's slot of rank d's staging rows (compute-only measurement: of its own)
                uint8_t *base = t->base[compute_only ? pe : d] + symm_off + static_cast<size_t>(pe) * mr * row_b;
                int rc = encode_2d(api, &mp.out[d], dt, base, n, rv_d, row_b, 64, 32);
                if (rc) return rc;
            }
            if (allreduce && rv_me > 0) {
                uint8_t *base = t->base[d] + symm_off + (static_cast<size_t>(R) * mr + static_cast<size_t>(pe) * mr) * row_b;
                int rc = encode_2d(api, &mp.fin[d], dt, base, n, rv_me, row_b, 64, 32);
                if (rc) return rc;
            }
        }
    }
    return CATCCOS_OK;
}

// Exchange format of the reduce family's partial tiles: fp16 by default (its 11-bit mantissa keeps the sum of
// up to seven rounded partials within the 1e-2 gate where bf16 partials do not; a partial beyond the fp16
// range is reported through the status words), CATCCOS_RS_EXCHANGE=native sends them in the output type,
// as the reference does (include/catccos/dgemm/kernel/matmul_reduce_scatter.hpp:314).
int rs_exchange_fp16() {
    const char *e = getenv("CATCCOS_RS_EXCHANGE");
    return (e && strcmp(e, "native") == 0) ? 0 : 1;
}

// one half of the (double-buffered) data region, rounded up to the 1024-byte alignment of the halves
static size_t dense_half_bytes(int op, int world, int m, int n, int k) {
    const size_t es = 2;
    size_t b = 0;
    switch (op) {
        case OP_AGMM: b = static_cast<size_t>(world) * m * k * es; break;
        case OP_MMRS:
        case OP_MMA2A: b = static_cast<size_t>(m) * n * es; break;
        case OP_MMAR: {
            const size_t mr = (m + world - 1) / world;
            b = 2 * static_cast<size_t>(world) * mr * n * es;
            break;
        }
    }
    return (b + 1023) / 1024 * 1024;
}

size_t dense_symmetric_bytes(int op, int world, int m, int n, int k) {
    if (world <= 1) return 0;
    return 2 * dense_half_bytes(op, world, m, n, k);
}

int launch_dense(int op, int dtype, cudaStream_t stream, uint32_t block_num, const DenseArgs *args, void *symmetric,
                 int m, int n, int k, int trans_a, int trans_b, int variant) {
    Team *t = team();
    if (!t) {
        set_error("symmetric heap not initialised (call catccos_shmem_init first)");
        return CATCCOS_ERR_NOT_INIT;
    }
    std::string why;
    const DriverApi *api = driver_api(&why);
    if (!api) {
        set_error("CUDA driver unavailable: %s", why.c_str());
        return CATCCOS_ERR_CUDA;
    }
    if (op != OP_AGMM && op != OP_MMRS && op != OP_MMAR && op != OP_MMA2A) {
        set_error("unknown dense operator %d", op);
        return CATCCOS_ERR_INVALID;
    }
    if (dtype != 1 && dtype != 27) {
        set_error("dense operators take FP16 (1) or BF16 (27), got %d", dtype);
        return CATCCOS_ERR_INVALID;
    }
    if (trans_a != 0) {
        set_error("transA=1 is not supported");
        return CATCCOS_ERR_INVALID;
    }
    if ((variant != AG_PUSH && variant != AG_REMOTE_READ && variant != AG_ALLTOALL) || (variant != AG_PUSH && op != OP_AGMM)) {
        set_error("data-flow variant %d does not exist for operator %d", variant, op);
        return CATCCOS_ERR_INVALID;
    }
    if (m <= 0 || n <= 0 || k <= 0 || (k % 8) != 0 || (n % 8) != 0) {
        set_error("unsupported shape m=%d n=%d k=%d (n and k must be positive multiples of 8)", m, n, k);
        return CATCCOS_ERR_INVALID;
    }
    const int R = t->n_pes;
    if ((op == OP_MMRS || op == OP_MMA2A) && (m % R) != 0) {
        set_error("matmul_reduce_scatter / matmul_alltoall need m (%d) divisible by the world size (%d)", m, R);
        return CATCCOS_ERR_INVALID;
    }
    const int n_local = t->emulated ? R : 1;
    const int nt = (n + BN - 1) / BN;
    const size_t need = dense_symmetric_bytes(op, R, m, n, k);
    uint64_t symm_off = 0;
    if (R > 1) {
        uint8_t *sp = static_cast<uint8_t *>(symmetric);
        uint8_t *b = t->base[t->my_pe];
        if (sp == nullptr || sp < b + kFlagBytes || sp + need > b + t->heap_bytes) {
            set_error("symmetric buffer %p (+%zu bytes) is not inside the symmetric heap", symmetric, need);
            return CATCCOS_ERR_INVALID;
        }
        symm_off = static_cast<uint64_t>(sp - b);
        if (symm_off % 1024 != 0) {
            set_error("symmetric buffer must be 1024-byte aligned");
            return CATCCOS_ERR_INVALID;
        }
        size_t flags = 0;
        if (op == OP_AGMM)      // arrival flags; remote read adds one "staged" flag per unit and source
            flags = static_cast<size_t>(R) * ((m + BM - 1) / BM) * kAgSubChunks * (variant == AG_REMOTE_READ ? 2 : 1);
        if (op == OP_MMRS || op == OP_MMA2A) flags = static_cast<size_t>(R) * ((m / R + BM - 1) / BM) * nt;
        if (op == OP_MMAR) flags = 2 * static_cast<size_t>(R) * (((m + R - 1) / R + BM - 1) / BM) * nt;
        if (kFlagOpBase + flags > kFlagWords) {
            set_error("shape needs %zu flags, the flag region holds %u", flags, kFlagWords - kFlagOpBase);
            return CATCCOS_ERR_INVALID;
        }
    }

    // which half of the region this launch uses, and how far the peers must have come (see next_slot)
    const uint32_t epoch = t->epoch + 1;
    uint64_t sig = slot_sig(0x44454E5345ull, static_cast<uint64_t>(op));
    sig = slot_sig(sig, static_cast<uint64_t>(dtype));
    sig = slot_sig(sig, static_cast<uint64_t>(m));
    sig = slot_sig(sig, static_cast<uint64_t>(n));
    sig = slot_sig(sig, static_cast<uint64_t>(k));
    sig = slot_sig(sig, symm_off);
    sig = slot_sig(sig, static_cast<uint64_t>(variant));
    const LaunchSlot slot = peek_slot(t, sig, epoch);
    if (R > 1) symm_off += static_cast<uint64_t>(slot.half) * dense_half_bytes(op, R, m, n, k);

    // the operators run on CTA pairs (cta_group::2) unless CATCCOS_TWO_CTA=0
    bool use_pair = true;
    if (const char *e = getenv("CATCCOS_TWO_CTA")) use_pair = atoi(e) != 0;
    bool wants_gather = false;
    for (int l = 0; l < n_local; ++l) wants_gather = wants_gather || args[l].gather_out != nullptr;
    if (!use_pair && (variant != AG_PUSH || wants_gather)) {
        set_error("the remote-read and gather-result variants of AllGather-Matmul exist in the CTA-pair kernel only "
                  "(unset CATCCOS_TWO_CTA=0)");
        return CATCCOS_ERR_INVALID;
    }
    if (!use_pair && op == OP_MMA2A) {
        set_error("Matmul-AllToAll exists in the CTA-pair kernel only (unset CATCCOS_TWO_CTA=0)");
        return CATCCOS_ERR_INVALID;
    }
    if (wants_gather && (op != OP_AGMM || variant == AG_ALLTOALL)) {
        set_error("only AllGather-Matmul returns the gathered A");
        return CATCCOS_ERR_INVALID;
    }
    FusedParams p;
    memset(&p, 0, sizeof(p));
    const CUtensorMapDataType dt = dtype == 27 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int a_rows = variant == AG_ALLTOALL ? R * m : m;   // rows of the caller's A
    for (int l = 0; l < n_local; ++l) {
        const DenseArgs &a = args[l];
        if (!a.A || !a.B || !a.C || (reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15) ||
            (reinterpret_cast<uintptr_t>(a.C) & 15)) {
            set_error("A, B and C must be non-null and 16-byte aligned");
            return CATCCOS_ERR_INVALID;
        }
        RankArgs &ra = p.ranks[l];
        int rc = encode_2d(api, &ra.tmA, dt, a.A, k, a_rows, static_cast<uint64_t>(k) * 2, BK, BM);
        if (rc) return rc;
        if (trans_b) {
            rc = encode_2d(api, &ra.tmB, dt, a.B, k, n, static_cast<uint64_t>(k) * 2, BK, use_pair ? 128 : BN);
        } else {
            rc = encode_2d(api, &ra.tmB, dt, a.B, n, k, static_cast<uint64_t>(n) * 2, 64, BK);
        }
        if (rc) return rc;
        if (op == OP_AGMM && R > 1) {
            const int pe = t->emulated ? l : t->my_pe;
            rc = encode_2d(api, &ra.tmAg, dt, t->base[pe] + symm_off, k, static_cast<uint64_t>(R) * m,
                           static_cast<uint64_t>(k) * 2, BK, BM);
            if (rc) return rc;
        } else {
            ra.tmAg = ra.tmA;
        }
        ra.A = a.A;
        ra.C = a.C;
        ra.gather_out = a.gather_out;
        if (a.gather_out && (reinterpret_cast<uintptr_t>(a.gather_out) & 15)) {
            set_error("the gathered-A output must be 16-byte aligned");
            return CATCCOS_ERR_INVALID;
        }
    }
    for (int pe = 0; pe < R; ++pe) p.heap_base[pe] = t->base[pe];
    p.symm_off = symm_off;
    p.world = R;
    p.rank_base = t->emulated ? 0 : t->my_pe;
    p.n_local = n_local;
    int per_rank = t->num_sms / n_local;
    if (block_num > 0 && static_cast<int>(block_num) < per_rank) per_rank = static_cast<int>(block_num);
    if (per_rank < 1) per_rank = 1;
    if (R > 1 && per_rank < 2) {
        set_error("fused operators need at least 2 CTAs per rank (blockNum=%u)", block_num);
        return CATCCOS_ERR_INVALID;
    }
    p.ctas_per_rank = per_rank;
    p.push_ctas = 0;
    if (op == OP_AGMM && R > 1) {
        // 0 (default): every CTA pushes next to its GEMM tiles; N > 0: N CTAs only push
        int pc = 0;
        if (const char *e = getenv("CATCCOS_PUSH_CTAS")) pc = atoi(e);
        if (pc > per_rank / 4) pc = per_rank / 4;
        if (pc < 0) pc = 0;
        p.push_ctas = pc;
    }
    p.M = m;
    p.N = n;
    p.K = k;
    p.epoch = epoch;
    p.entered_need = slot.entered_need;
    p.compute_only = (t->debug_flags & 1u) ? 1 : 0;
    p.timeout_ns = t->timeout_ns;
    p.status = t->status_dev;
    p.rs_fp16 = op == OP_MMA2A ? 0 : rs_exchange_fp16();      // rows that are only moved keep the output type
    // all-gather through the NVSwitch multicast view when the team has one (plain AllGather-Matmul only)
    p.mc_base = (op == OP_AGMM && variant == AG_PUSH && !wants_gather && R > 1 && !t->emulated) ? t->mc_base : nullptr;
    p.ag_pull = variant == AG_REMOTE_READ ? 1 : 0;
    p.ag_a2a = variant == AG_ALLTOALL ? 1 : 0;
    p.sched = t->sched_dev;
    p.trace = t->trace_dev;

    const bool coop = n_local > 1;
    const bool bf16 = dtype == 27;
    const bool b_mn = trans_b == 0;
    if (use_pair && per_rank < 2) {
        set_error("the CTA-pair kernel needs at least 2 CTAs per rank");
        return CATCCOS_ERR_INVALID;
    }
    // output tensor maps of the pair reduce-scatter kernel (see RsMaps)
    static thread_local RsMapsAll maps;
    if (use_pair && op != OP_AGMM) {
        void *outs[kMaxRanks];
        for (int l = 0; l < n_local; ++l) outs[l] = args[l].C;
        int rc = encode_rs_maps(api, t, &maps, op, dt, outs, n_local, m, n, symm_off, p.compute_only != 0);
        if (rc) return rc;
    }
    commit_slot(t, sig, epoch, slot);
    if (use_pair) {
        p.ctas_per_rank = per_rank & ~1;
        p.push_ctas = 0;
        // L2 grouping of the AllGather-Matmul tile order: rows of A per group from an L2 budget
        // (CATCCOS_AG_GROUP overrides the choice, CATCCOS_AG_L2_MB the budget)
        long long l2_mb = 88;
        if (const char *e = getenv("CATCCOS_AG_L2_MB")) l2_mb = atoll(e) > 0 ? atoll(e) : l2_mb;
        p.ag_group = ag_order_group_rows(256ll * k * 2, p.ctas_per_rank / 2, l2_mb << 20);
        const int mt2 = (m + 2 * BM - 1) / (2 * BM);
        if (R > 1 && p.ag_group > mt2) p.ag_group = p.ag_group / mt2 * mt2;      // whole sources per group
        if (const char *e = getenv("CATCCOS_AG_GROUP")) {
            if (atoi(e) > 0) p.ag_group = atoi(e);
        }
        const int g2 = p.ctas_per_rank * n_local;
        if (bf16)
            return b_mn ? launch_pair<__nv_bfloat16, true>(op, p, maps, g2, coop, stream)
                        : launch_pair<__nv_bfloat16, false>(op, p, maps, g2, coop, stream);
        return b_mn ? launch_pair<__half, true>(op, p, maps, g2, coop, stream) : launch_pair<__half, false>(op, p, maps, g2, coop, stream);
    }
    const int grid = per_rank * n_local;
    switch (op) {
        case OP_AGMM: return launch_t<OP_AGMM>(p, grid, coop, stream, bf16, b_mn);
        case OP_MMRS: return launch_t<OP_MMRS>(p, grid, coop, stream, bf16, b_mn);
        default: return launch_t<OP_MMAR>(p, grid, coop, stream, bf16, b_mn);
    }
}

}  // namespace cb
