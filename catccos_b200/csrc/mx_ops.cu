// Host launcher of the MXFP8 AllGather-Matmul.
#include "mx_ops.h"

#include <string.h>

#include "mx_gemm.cuh"
#include "mx_pair.cuh"
#include "mx_pair_rs.cuh"
#include "dense_ops.h"
#include <stdlib.h>
#include "mx_quant.h"

namespace cb {

static int encode_u8(const DriverApi *api, CUtensorMap *tm, const void *base, uint64_t inner, uint64_t outer,
                     uint32_t box_inner, uint32_t box_outer) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = api->TensorMapEncodeTiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides,
                                           box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (u8) failed: %d (base=%p inner=%llu outer=%llu)", static_cast<int>(r), base,
                  (unsigned long long)inner, (unsigned long long)outer);
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

// scale atoms as a 2-D tensor: rows of 128 u32 (= one 512-byte atom), one atom per load
static int encode_atoms(const DriverApi *api, CUtensorMap *tm, const void *base, uint64_t n_atoms) {
    cuuint64_t dims[2] = {128, n_atoms};
    cuuint64_t strides[1] = {512};
    cuuint32_t box[2] = {128, 1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = api->TensorMapEncodeTiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(base), dims, strides,
                                           box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (scale atoms) failed: %d (base=%p atoms=%llu)", static_cast<int>(r), base,
                  (unsigned long long)n_atoms);
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// one half of the (double-buffered) gathered region: codes (k bytes per row; k/2 for 4-bit codes), then scale atoms
static size_t mx_ag_half_bytes(int world, int m, int k, int fmt = MX_FP8) {
    const size_t row = fmt == MX_FP4 ? k / 2 : k;
    const size_t data = align_up(static_cast<size_t>(world) * m * row, 1024);
    return align_up(data + static_cast<size_t>(world) * sf_atoms_bytes(m, k), 1024);
}

size_t mx_ag_symmetric_bytes(int world, int m, int n, int k, int fmt) {
    (void)n;
    if (world <= 1) return 0;
    return 2 * mx_ag_half_bytes(world, m, k, fmt);
}

size_t mx_ag_workspace_bytes(int m, int n, int k) {
    return align_up(sf_atoms_bytes(m, k), 1024) + align_up(sf_atoms_bytes(n, k), 1024);
}

template <typename TOut, bool B_MN>
static int launch_pair_k(const MxParams &p, int grid, bool coop, cudaStream_t stream) {
    auto kern = mx_pair_agmm_kernel<TOut, B_MN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMxPairSmemBytes);
    if (e == cudaSuccess) {
        if (coop) {
            void *args[] = {const_cast<MxParams *>(&p)};
            e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(kern), dim3(grid), dim3(kMxPairThreads), args,
                                            kMxPairSmemBytes, stream);
        } else {
            kern<<<grid, kMxPairThreads, kMxPairSmemBytes, stream>>>(p);
            e = cudaGetLastError();
        }
    }
    if (e != cudaSuccess) {
        set_error("MX pair kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

template <typename TOut, bool B_MN, int FMT = MX_FP8>
static int launch_k(const MxParams &p, int grid, bool coop, cudaStream_t stream) {
    auto kern = mx_allgather_gemm_kernel<TOut, B_MN, FMT>;
    constexpr int kSmem = MxCfg<FMT>::kSmemBytes;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e == cudaSuccess) {
        if (coop) {
            void *args[] = {const_cast<MxParams *>(&p)};
            e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(kern), dim3(grid), dim3(kGemmThreads), args,
                                            kSmem, stream);
        } else {
            kern<<<grid, kGemmThreads, kSmem, stream>>>(p);
            e = cudaGetLastError();
        }
    }
    if (e != cudaSuccess) {
        set_error("MX kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

int launch_mx_allgather_matmul(int out_dtype, cudaStream_t stream, uint32_t block_num, const MxAgArgs *args,
                               void *symmetric, int m, int n, int k, int trans_b, int fmt) {
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
    if (out_dtype != 1 && out_dtype != 27) {
        set_error("MXFP8 AllGather-Matmul writes FP16 (1) or BF16 (27), got %d", out_dtype);
        return CATCCOS_ERR_INVALID;
    }
    if (m <= 0 || n <= 0 || k <= 0 || (k % 32) != 0 || (n % 16) != 0) {
        set_error("unsupported shape m=%d n=%d k=%d (k multiple of 32, n multiple of 16)", m, n, k);
        return CATCCOS_ERR_INVALID;
    }
    if (fmt != MX_FP8 && fmt != MX_FP4) {
        set_error("unknown block-scaled format %d", fmt);
        return CATCCOS_ERR_INVALID;
    }
    if (fmt == MX_FP4 && (!trans_b || (k % 64) != 0)) {
        set_error("MXFP4 AllGather-Matmul needs K-major operands (transB = 1) and k a multiple of 64 (k=%d transB=%d)", k, trans_b);
        return CATCCOS_ERR_INVALID;
    }
    const int kbytes = fmt == MX_FP4 ? k / 2 : k;      // bytes of one operand row
    const int R = t->n_pes;
    const int n_local = t->emulated ? R : 1;
    const int mt = (m + BM - 1) / BM;
    const size_t need = mx_ag_symmetric_bytes(R, m, n, k, fmt);
    uint64_t symm_off = 0, sf_off = 0;
    const uint32_t epoch = t->epoch + 1;
    LaunchSlot slot{0, epoch};
    uint64_t sig = 0;
    if (R > 1) {
        uint8_t *sp = static_cast<uint8_t *>(symmetric);
        uint8_t *b = t->base[t->my_pe];
        if (sp == nullptr || sp < b + kFlagBytes || sp + need > b + t->heap_bytes || ((sp - b) % 1024) != 0) {
            set_error("symmetric buffer %p (+%zu bytes) is not a 1024-aligned range of the symmetric heap", symmetric, need);
            return CATCCOS_ERR_INVALID;
        }
        symm_off = static_cast<uint64_t>(sp - b);
        sig = slot_sig(0x4D584147ull + static_cast<uint64_t>(fmt), static_cast<uint64_t>(m));
        sig = slot_sig(sig, static_cast<uint64_t>(n));
        sig = slot_sig(sig, static_cast<uint64_t>(k));
        sig = slot_sig(sig, symm_off);
        slot = peek_slot(t, sig, epoch);      // which half of the region this launch uses
        symm_off += static_cast<uint64_t>(slot.half) * mx_ag_half_bytes(R, m, k, fmt);
        sf_off = symm_off + align_up(static_cast<size_t>(R) * m * kbytes, 1024);
        if (kFlagOpBase + static_cast<size_t>(R) * mt * kMxFlagsPerChunk > kFlagWords) {
            set_error("shape needs more flags than the flag region holds");
            return CATCCOS_ERR_INVALID;
        }
    }
    bool use_pair = true;      // CTA pairs (cta_group::2) unless CATCCOS_TWO_CTA=0
    if (const char *e = getenv("CATCCOS_TWO_CTA")) use_pair = atoi(e) != 0;
    const int kb4 = (k + 127) / 128;
    MxParams p;
    memset(&p, 0, sizeof(p));
    const int kblocks = k / 32;
    const int a_ld = (kblocks + 1) / 2 * 2;
    for (int l = 0; l < n_local; ++l) {
        const MxAgArgs &a = args[l];
        if (!a.A || !a.B || !a.C || !a.a_scale || !a.b_scale || !a.workspace ||
            (reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15) ||
            (reinterpret_cast<uintptr_t>(a.C) & 15) || (reinterpret_cast<uintptr_t>(a.workspace) & 15)) {
            set_error("A, B, C, both scale tensors and the workspace must be non-null (16-byte aligned data)");
            return CATCCOS_ERR_INVALID;
        }
        uint8_t *sfa = a.workspace;
        uint8_t *sfb = a.workspace + align_up(sf_atoms_bytes(m, k), 1024);
        int rc = sf_to_atoms_launch(stream, a.a_scale, 0, m, kblocks, a_ld, sfa);
        if (rc) return rc;
        rc = trans_b ? sf_to_atoms_launch(stream, a.b_scale, 0, n, kblocks, a_ld, sfb)
                     : sf_to_atoms_launch(stream, a.b_scale, 1, n, kblocks, 0, sfb);
        if (rc) return rc;
        MxRankArgs &ra = p.ranks[l];
        if ((rc = encode_u8(api, &ra.tmA, a.A, kbytes, m, MX_BK, BM))) return rc;
        rc = trans_b ? encode_u8(api, &ra.tmB, a.B, kbytes, n, MX_BK, use_pair ? 128 : BN)
                     : encode_u8(api, &ra.tmB, a.B, n, k, 128, MX_BK);
        if (rc) return rc;
        if (use_pair) {
            if ((rc = encode_atoms(api, &ra.tmSfa, sfa, static_cast<uint64_t>(mt) * kb4))) return rc;
            if ((rc = encode_atoms(api, &ra.tmSfb, sfb, static_cast<uint64_t>((n + 127) / 128) * kb4))) return rc;
            const int pe2 = t->emulated ? l : t->my_pe;
            if (R > 1) {
                if ((rc = encode_atoms(api, &ra.tmSfag, t->base[pe2] + sf_off, static_cast<uint64_t>(R) * mt * kb4))) return rc;
            } else {
                ra.tmSfag = ra.tmSfa;
            }
        }
        if (R > 1) {
            const int pe = t->emulated ? l : t->my_pe;
            if ((rc = encode_u8(api, &ra.tmAg, t->base[pe] + symm_off, kbytes, static_cast<uint64_t>(R) * m, MX_BK, BM)))
                return rc;
        } else {
            ra.tmAg = ra.tmA;
        }
        ra.A = a.A;
        ra.sfa = sfa;
        ra.sfb = sfb;
        ra.C = a.C;
    }
    for (int pe = 0; pe < R; ++pe) p.heap_base[pe] = t->base[pe];
    p.symm_off = symm_off;
    p.sf_off = sf_off;
    p.world = R;
    p.rank_base = t->emulated ? 0 : t->my_pe;
    p.n_local = n_local;
    int per_rank = t->num_sms / n_local;
    if (block_num > 0 && static_cast<int>(block_num) < per_rank) per_rank = static_cast<int>(block_num);
    if (per_rank < 1) per_rank = 1;
    p.ctas_per_rank = per_rank;
    p.M = m;
    p.N = n;
    p.K = k;
    p.fp4 = fmt == MX_FP4 ? 1 : 0;
    p.epoch = epoch;
    p.entered_need = slot.entered_need;
    p.compute_only = (t->debug_flags & 1u) ? 1 : 0;
    p.timeout_ns = t->timeout_ns;
    p.status = t->status_dev;
    p.trace = t->trace_dev;
    const bool coop = n_local > 1;
    const bool b_mn = trans_b == 0;
    commit_slot(t, sig, epoch, slot);
    if (use_pair && per_rank >= 2) {
        p.ctas_per_rank = per_rank & ~1;
        const int g2 = p.ctas_per_rank * n_local;
        if (out_dtype == 27)
            return b_mn ? launch_pair_k<__nv_bfloat16, true>(p, g2, coop, stream) : launch_pair_k<__nv_bfloat16, false>(p, g2, coop, stream);
        return b_mn ? launch_pair_k<__half, true>(p, g2, coop, stream) : launch_pair_k<__half, false>(p, g2, coop, stream);
    }
    const int grid = per_rank * n_local;
    if (fmt == MX_FP4)
        return out_dtype == 27 ? launch_k<__nv_bfloat16, false, MX_FP4>(p, grid, coop, stream)
                               : launch_k<__half, false, MX_FP4>(p, grid, coop, stream);
    if (out_dtype == 27)
        return b_mn ? launch_k<__nv_bfloat16, true>(p, grid, coop, stream) : launch_k<__nv_bfloat16, false>(p, grid, coop, stream);
    return b_mn ? launch_k<__half, true>(p, grid, coop, stream) : launch_k<__half, false>(p, grid, coop, stream);
}

template <typename TOut, bool B_MN, int FMT = MX_FP8>
static int launch_rs_k(const MxRsParams &p, const RsMapsAll &maps, int grid, bool coop, cudaStream_t stream) {
    auto kern = mx_pair_rs_kernel<TOut, B_MN, FMT>;
    constexpr int kSmem = FMT == MX_FP4 ? kMxRsSmemBytesFp4 : kMxRsSmemBytes;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e == cudaSuccess) {
        if (coop) {
            void *args[] = {const_cast<MxRsParams *>(&p), const_cast<RsMapsAll *>(&maps)};
            e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(kern), dim3(grid), dim3(kGemmThreads), args,
                                            kSmem, stream);
        } else {
            kern<<<grid, kGemmThreads, kSmem, stream>>>(p, maps);
            e = cudaGetLastError();
        }
    }
    if (e != cudaSuccess) {
        set_error("MX reduce-scatter kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

int launch_mx_matmul_reduce_scatter(int out_dtype, int code_format, cudaStream_t stream, uint32_t block_num,
                                    const MxAgArgs *args, void *symmetric, int m, int n, int k, int trans_b, int alltoall) {
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
    if (out_dtype != 1 && out_dtype != 27) {
        set_error("MXFP8 Matmul-ReduceScatter writes FP16 (1) or BF16 (27), got %d", out_dtype);
        return CATCCOS_ERR_INVALID;
    }
    if (code_format != 0 && code_format != 1 && code_format != 2) {
        set_error("code format must be 0 (e4m3), 1 (e5m2) or 2 (e2m1, MXFP4), got %d", code_format);
        return CATCCOS_ERR_INVALID;
    }
    const bool fp4 = code_format == 2;
    if (fp4 && (!trans_b || (k % 64) != 0)) {
        set_error("MXFP4 operands are K-major (transB = 1) with k a multiple of 64 (k=%d transB=%d)", k, trans_b);
        return CATCCOS_ERR_INVALID;
    }
    const int kbytes = fp4 ? k / 2 : k;
    const int R = t->n_pes;
    if (m <= 0 || n <= 0 || k <= 0 || (k % 32) != 0 || (n % 16) != 0 || (m % R) != 0 || ((m / R) % BM) != 0) {
        set_error("unsupported shape m=%d n=%d k=%d for %d ranks (k multiple of 32, n multiple of 16, m/ranks multiple of %d)",
                  m, n, k, R, BM);
        return CATCCOS_ERR_INVALID;
    }
    const int n_local = t->emulated ? R : 1;
    const int nt = (n + BN - 1) / BN;
    const size_t need = dense_symmetric_bytes(OP_MMRS, R, m, n, k);
    uint64_t symm_off = 0;
    const uint32_t epoch = t->epoch + 1;
    LaunchSlot slot{0, epoch};
    uint64_t sig = 0;
    if (R > 1) {
        uint8_t *sp = static_cast<uint8_t *>(symmetric);
        uint8_t *b = t->base[t->my_pe];
        if (sp == nullptr || sp < b + kFlagBytes || sp + need > b + t->heap_bytes || ((sp - b) % 1024) != 0) {
            set_error("symmetric buffer %p (+%zu bytes) is not a 1024-aligned range of the symmetric heap", symmetric, need);
            return CATCCOS_ERR_INVALID;
        }
        symm_off = static_cast<uint64_t>(sp - b);
        if (kFlagOpBase + static_cast<size_t>(R) * ((m / R) / BM) * nt > kFlagWords) {
            set_error("shape needs more flags than the flag region holds");
            return CATCCOS_ERR_INVALID;
        }
        sig = slot_sig(0x4D585253ull + static_cast<uint64_t>(code_format) * 16 + (alltoall ? 1 : 0), static_cast<uint64_t>(m));
        sig = slot_sig(sig, static_cast<uint64_t>(n));
        sig = slot_sig(sig, static_cast<uint64_t>(k));
        sig = slot_sig(sig, symm_off);
        slot = peek_slot(t, sig, epoch);
        symm_off += static_cast<uint64_t>(slot.half) * (need / 2);
    }
    int per_rank = t->num_sms / n_local;
    if (block_num > 0 && static_cast<int>(block_num) < per_rank) per_rank = static_cast<int>(block_num);
    per_rank &= ~1;
    if (per_rank < 2) {
        set_error("the CTA-pair kernel needs at least 2 CTAs per rank (blockNum=%u)", block_num);
        return CATCCOS_ERR_INVALID;
    }
    const int kb4 = (k + 127) / 128;
    const int kblocks = k / 32;
    const int a_ld = (kblocks + 1) / 2 * 2;
    const int mt = (m + BM - 1) / BM;
    static thread_local MxRsParams p;
    memset(&p, 0, sizeof(p));
    void *outs[kMaxRanks];
    for (int l = 0; l < n_local; ++l) {
        const MxAgArgs &a = args[l];
        if (!a.A || !a.B || !a.C || !a.a_scale || !a.b_scale || !a.workspace ||
            (reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15) ||
            (reinterpret_cast<uintptr_t>(a.C) & 15) || (reinterpret_cast<uintptr_t>(a.workspace) & 15)) {
            set_error("A, B, C, both scale tensors and the workspace must be non-null (16-byte aligned data)");
            return CATCCOS_ERR_INVALID;
        }
        uint8_t *sfa = a.workspace;
        uint8_t *sfb = a.workspace + align_up(sf_atoms_bytes(m, k), 1024);
        int rc = sf_to_atoms_launch(stream, a.a_scale, 0, m, kblocks, a_ld, sfa);
        if (rc) return rc;
        rc = trans_b ? sf_to_atoms_launch(stream, a.b_scale, 0, n, kblocks, a_ld, sfb)
                     : sf_to_atoms_launch(stream, a.b_scale, 1, n, kblocks, 0, sfb);
        if (rc) return rc;
        MxRankArgs &ra = p.ranks[l];
        if ((rc = encode_u8(api, &ra.tmA, a.A, kbytes, m, MX_BK, BM))) return rc;
        rc = trans_b ? encode_u8(api, &ra.tmB, a.B, kbytes, n, MX_BK, 128) : encode_u8(api, &ra.tmB, a.B, n, k, 128, MX_BK);
        if (rc) return rc;
        if ((rc = encode_atoms(api, &ra.tmSfa, sfa, static_cast<uint64_t>(mt) * kb4))) return rc;
        if ((rc = encode_atoms(api, &ra.tmSfb, sfb, static_cast<uint64_t>((n + 127) / 128) * kb4))) return rc;
        ra.tmAg = ra.tmA;
        ra.tmSfag = ra.tmSfa;
        ra.A = a.A;
        ra.sfa = sfa;
        ra.sfb = sfb;
        ra.C = a.C;
        outs[l] = a.C;
    }
    const bool compute_only = (t->debug_flags & 1u) != 0;
    static thread_local RsMapsAll maps;
    const CUtensorMapDataType dt = out_dtype == 27 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    int rc = encode_rs_maps(api, t, &maps, alltoall ? OP_MMA2A : OP_MMRS, dt, outs, n_local, m, n, symm_off, compute_only);
    if (rc) return rc;
    for (int pe = 0; pe < R; ++pe) p.heap_base[pe] = t->base[pe];
    p.symm_off = symm_off;
    p.world = R;
    p.rank_base = t->emulated ? 0 : t->my_pe;
    p.n_local = n_local;
    p.ctas_per_rank = per_rank;
    p.M = m;
    p.N = n;
    p.K = k;
    p.fmt_bits = code_format == 1 ? ((1u << 7) | (1u << 10)) : 0u;
    p.a2a = alltoall ? 1 : 0;
    p.epoch = epoch;
    p.entered_need = slot.entered_need;
    p.compute_only = compute_only ? 1 : 0;
    p.rs_fp16 = alltoall ? 0 : rs_exchange_fp16();      // rows that are only moved keep the output type
    p.timeout_ns = t->timeout_ns;
    p.status = t->status_dev;
    p.trace = t->trace_dev;
    commit_slot(t, sig, epoch, slot);
    const bool coop = n_local > 1;
    const bool b_mn = trans_b == 0;
    const int grid = per_rank * n_local;
    if (fp4)
        return out_dtype == 27 ? launch_rs_k<__nv_bfloat16, false, MX_FP4>(p, maps, grid, coop, stream)
                               : launch_rs_k<__half, false, MX_FP4>(p, maps, grid, coop, stream);
    if (out_dtype == 27)
        return b_mn ? launch_rs_k<__nv_bfloat16, true>(p, maps, grid, coop, stream)
                    : launch_rs_k<__nv_bfloat16, false>(p, maps, grid, coop, stream);
    return b_mn ? launch_rs_k<__half, true>(p, maps, grid, coop, stream) : launch_rs_k<__half, false>(p, maps, grid, coop, stream);
}

}  // namespace cb
