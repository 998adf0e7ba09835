// Host orchestration of the MoE dispatch -> grouped GEMM -> SwiGLU -> grouped GEMM -> combine operator.
#include "moe_ops.h"

#include <stdlib.h>
#include <string.h>

#include "moe_gemm.cuh"
#include "moe_pair.cuh"
#include "mx_quant.h"

namespace cb {

static cudaEvent_t g_stage_ev[12] = {};     // debug flag 2: events between the stages of the last MoE launch
static int g_stage_count = 0;


static size_t up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int moe_rows_cap(int world, int m, int top_k, int experts_per_rank) {
    // Receive rows per rank.  The worst case (every token of every rank routed to one rank) is
    // world * m * topK; by default room is kept for twice the balanced load (at least 16 Ki rows),
    // never more than the worst case, plus the 128-row alignment of every local expert's segment.
    double factor = 2.0;
    if (const char *e = getenv("CATCCOS_MOE_CAPACITY_FACTOR")) {
        const double f = atof(e);
        if (f >= 1.0) factor = f;
    }
    const long long worst = static_cast<long long>(world) * m * top_k;
    long long cap = static_cast<long long>(factor * m * top_k);
    if (cap < 16384) cap = 16384;
    if (cap > worst) cap = worst;
    cap += static_cast<long long>(experts_per_rank) * 128;
    return static_cast<int>(up(static_cast<size_t>(cap), 128));
}

struct MoeSizes {
    int rows_cap, sld1, sld2;
    size_t counts, recv_codes, recv_scale, combine;                 // symmetric
    size_t idx, meta, recv_atoms, w1_atoms, w2_atoms, act_codes, act_atoms;   // workspace
};

static MoeSizes moe_sizes(int world, int m, int k, int n, int top_k, int experts) {
    MoeSizes z;
    const int el = experts / world;
    z.rows_cap = moe_rows_cap(world, m, top_k, el);
    z.sld1 = (k / 32 + 1) / 2 * 2;
    z.sld2 = ((n / 2) / 32 + 1) / 2 * 2;
    z.counts = up(static_cast<size_t>(world) * experts * 4, 1024);
    z.recv_codes = up(static_cast<size_t>(z.rows_cap) * k, 1024);
    z.recv_scale = up(static_cast<size_t>(z.rows_cap) * z.sld1, 1024);
    z.combine = up(static_cast<size_t>(m) * top_k * k * 2, 1024);
    z.idx = up(static_cast<size_t>(m) * top_k * 4, 1024);
    z.meta = up(sizeof(MoeMeta), 1024);
    z.recv_atoms = up(sf_atoms_bytes(z.rows_cap, k), 1024);
    z.w1_atoms = up(sf_atoms_bytes(el * n, k), 1024);
    z.w2_atoms = up(sf_atoms_bytes(el * k, n / 2), 1024);
    z.act_codes = up(static_cast<size_t>(z.rows_cap) * (n / 2), 1024);
    z.act_atoms = up(sf_atoms_bytes(z.rows_cap, n / 2), 1024);
    return z;
}

size_t moe_symmetric_bytes(int world, int m, int k, int n, int top_k, int experts) {
    const MoeSizes z = moe_sizes(world, m, k, n, top_k, experts);
    return z.counts + z.recv_codes + z.recv_scale + z.combine;
}
size_t moe_workspace_bytes(int world, int m, int k, int n, int top_k, int experts) {
    const MoeSizes z = moe_sizes(world, m, k, n, top_k, experts);
    return z.idx + z.meta + z.recv_atoms + z.w1_atoms + z.w2_atoms + z.act_codes + z.act_atoms;
}

static int encode_u8(const DriverApi *api, CUtensorMap *tm, const void *base, uint64_t inner, uint64_t outer) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner};
    cuuint32_t box[2] = {128, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = api->TensorMapEncodeTiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides,
                                           box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (MoE) failed: %d", static_cast<int>(r));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

template <int MODE, typename TOut, bool B_MN>
int launch_pair_gemm(const MoePairParams &p, cudaStream_t stream) {
    auto kern = moe_pair_gemm_kernel<MODE, TOut, B_MN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMoePairSmemBytes);
    if (e == cudaSuccess) {
        kern<<<p.ctas_per_rank * p.n_local, kMoePairThreads, kMoePairSmemBytes, stream>>>(p);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        set_error("MoE pair grouped GEMM launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

template <int MODE>
static int launch_gemm(const MoeGemmParams &p, cudaStream_t stream) {
    auto kern = moe_grouped_gemm_kernel<MODE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMoeSmemBytes);
    if (e == cudaSuccess) {
        kern<<<p.ctas_per_rank * p.n_local, kGemmThreads, kMoeSmemBytes, stream>>>(p);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        set_error("MoE grouped GEMM launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

int launch_moe_dispatch_ffn_combine(cudaStream_t stream, uint32_t block_num, const MoeArgs *args, void *symmetric,
                                    int m, int k, int n, int top_k, int experts) {
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
    const int R = t->n_pes;
    // same shape rule as the reference operator (ascend950_dispatch_ffn_combine_host.h:183)
    if (m <= 0 || k <= 0 || n <= 0 || (k % 256) != 0 || (n % 512) != 0) {
        set_error("MXFP8 dispatch_ffn_combine requires K %% 256 == 0 and N %% 512 == 0 (m=%d k=%d n=%d)", m, k, n);
        return CATCCOS_ERR_INVALID;
    }
    if (experts <= 0 || experts % R != 0 || experts > kMoeMaxExperts || experts / R > kMoeMaxLocalExperts ||
        top_k <= 0 || top_k > 16 || top_k > experts) {
        set_error("unsupported expert setup: experts=%d (max %d, divisible by world %d, at most %d per rank) topK=%d (max 16)",
                  experts, kMoeMaxExperts, R, kMoeMaxLocalExperts, top_k);
        return CATCCOS_ERR_INVALID;
    }
    const int el = experts / R;
    const int n_local = t->emulated ? R : 1;
    const MoeSizes z = moe_sizes(R, m, k, n, top_k, experts);
    const size_t need = z.counts + z.recv_codes + z.recv_scale + z.combine;
    uint8_t *sp = static_cast<uint8_t *>(symmetric);
    uint8_t *hb = t->base[t->my_pe];
    if (sp == nullptr || sp < hb + kFlagBytes || sp + need > hb + t->heap_bytes || ((sp - hb) % 1024) != 0) {
        set_error("symmetric buffer %p (+%zu bytes) is not a 1024-aligned range of the symmetric heap", symmetric, need);
        return CATCCOS_ERR_INVALID;
    }
    const uint64_t off0 = static_cast<uint64_t>(sp - hb);

    MoeParams p;
    memset(&p, 0, sizeof(p));
    p.lay.counts_off = off0;
    p.lay.recv_codes_off = off0 + z.counts;
    p.lay.recv_scale_off = p.lay.recv_codes_off + z.recv_codes;
    p.lay.combine_off = p.lay.recv_scale_off + z.recv_scale;
    p.lay.rows_cap = z.rows_cap;
    p.lay.scale_ld = z.sld1;
    for (int pe = 0; pe < R; ++pe) p.heap_base[pe] = t->base[pe];
    p.world = R;
    p.rank_base = t->emulated ? 0 : t->my_pe;
    p.n_local = n_local;
    int per_rank = t->num_sms / n_local;
    if (block_num > 0 && static_cast<int>(block_num) < per_rank) per_rank = static_cast<int>(block_num);
    if (per_rank < 1) per_rank = 1;
    p.ctas_per_rank = per_rank;
    p.m = m;
    p.K = k;
    p.N = n;
    p.top_k = top_k;
    p.experts = experts;
    p.experts_per_rank = el;
    p.epoch = ++t->epoch;
    p.timeout_ns = t->timeout_ns;
    p.status = t->status_dev;

    MoeGemmParams g1, g2;
    memset(&g1, 0, sizeof(g1));
    for (int pe = 0; pe < R; ++pe) g1.heap_base[pe] = t->base[pe];
    g1.combine_off = p.lay.combine_off;
    g1.world = R;
    g1.rank_base = p.rank_base;
    g1.n_local = n_local;
    g1.ctas_per_rank = per_rank;
    g1.experts = experts;
    g1.experts_per_rank = el;
    g1.epoch = p.epoch;
    g1.timeout_ns = p.timeout_ns;
    g1.status = p.status;
    g2 = g1;
    g1.Kin = k;
    g1.Nw = n;
    g1.counter_slot = 1;
    g2.Kin = n / 2;
    g2.Nw = k;
    g2.counter_slot = 2;

    // the grouped GEMMs run on CTA pairs (cta_group::2) unless CATCCOS_TWO_CTA=0
    bool use_pair = per_rank >= 2;
    if (const char *e = getenv("CATCCOS_TWO_CTA")) use_pair = use_pair && atoi(e) != 0;
    static thread_local MoePairParams q1, q2;
    memset(&q1, 0, sizeof(q1));
    for (int pe = 0; pe < R; ++pe) q1.heap_base[pe] = t->base[pe];
    q1.combine_off = p.lay.combine_off;
    q1.world = R;
    q1.rank_base = p.rank_base;
    q1.n_local = n_local;
    q1.ctas_per_rank = per_rank & ~1;
    q1.rows_cap = z.rows_cap;
    q1.experts = experts;
    q1.experts_per_rank = el;
    q1.epoch = p.epoch;
    q1.timeout_ns = p.timeout_ns;
    q1.status = p.status;
    q2 = q1;
    q1.Kin = k;
    q1.Nw = n;
    q1.counter_slot = 1;
    q2.Kin = n / 2;
    q2.Nw = k;
    q2.counter_slot = 2;

    struct Ws { uint8_t *recv_atoms, *w1_atoms, *w2_atoms, *act_codes, *act_atoms; } ws[kMaxRanks];
    for (int l = 0; l < n_local; ++l) {
        const MoeArgs &a = args[l];
        if (!a.x || !a.w1 || !a.out || !a.w2 || !a.expert_idx || !a.probs || !a.w1_scale || !a.w2_scale || !a.workspace ||
            (reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.out) & 15) ||
            (reinterpret_cast<uintptr_t>(a.w1) & 15) || (reinterpret_cast<uintptr_t>(a.w2) & 15) ||
            (reinterpret_cast<uintptr_t>(a.workspace) & 255)) {
            set_error("dispatch_ffn_combine: every operand must be non-null; tensors 16-byte, workspace 256-byte aligned");
            return CATCCOS_ERR_INVALID;
        }
        uint8_t *w = a.workspace;
        MoeRankArgs &ra = p.ranks[l];
        ra.x = a.x;
        ra.expert_idx = a.expert_idx;
        ra.probs = a.probs;
        ra.out = a.out;
        ra.expanded_row_idx = reinterpret_cast<int *>(w);
        w += z.idx;
        ra.meta = reinterpret_cast<MoeMeta *>(w);
        w += z.meta;
        ws[l].recv_atoms = w;
        w += z.recv_atoms;
        ws[l].w1_atoms = w;
        w += z.w1_atoms;
        ws[l].w2_atoms = w;
        w += z.w2_atoms;
        ws[l].act_codes = w;
        w += z.act_codes;
        ws[l].act_atoms = w;
        const int pe = t->emulated ? l : t->my_pe;
        uint8_t *recv_codes = t->base[pe] + p.lay.recv_codes_off;
        int rc;
        MoeGemmRankArgs &r1 = g1.ranks[l];
        if ((rc = encode_u8(api, &r1.tmA, recv_codes, k, z.rows_cap))) return rc;
        if ((rc = encode_u8(api, &r1.tmB, a.w1, k, static_cast<uint64_t>(el) * n))) return rc;
        r1.sfa = ws[l].recv_atoms;
        r1.sfb = ws[l].w1_atoms;
        r1.act_codes = ws[l].act_codes;
        r1.act_sf = ws[l].act_atoms;
        r1.meta = ra.meta;
        MoeGemmRankArgs &r2 = g2.ranks[l];
        if ((rc = encode_u8(api, &r2.tmA, ws[l].act_codes, n / 2, z.rows_cap))) return rc;
        if ((rc = encode_u8(api, &r2.tmB, a.w2, n / 2, static_cast<uint64_t>(el) * k))) return rc;
        r2.sfa = ws[l].act_atoms;
        r2.sfb = ws[l].w2_atoms;
        r2.act_codes = nullptr;
        r2.act_sf = nullptr;
        r2.meta = ra.meta;
        if (use_pair) {
            MoePairRankArgs &p1 = q1.ranks[l];
            p1.tmA = r1.tmA;
            p1.tmB = r1.tmB;
            p1.sfa = ws[l].recv_atoms;
            p1.sfb = ws[l].w1_atoms;
            p1.act_codes = ws[l].act_codes;
            p1.act_sf = ws[l].act_atoms;
            p1.meta = ra.meta;
            MoePairRankArgs &p2 = q2.ranks[l];
            p2.tmA = r2.tmA;
            p2.tmB = r2.tmB;
            p2.sfa = ws[l].act_atoms;
            p2.sfb = ws[l].w2_atoms;
            p2.act_codes = nullptr;
            p2.act_sf = nullptr;
            p2.meta = ra.meta;
        }
    }

    // debug flag 2: CUDA events between the stages of this launch (read back with moe_stage_ms)
    const bool timed = (t->debug_flags & 2u) != 0;
    int stage = 0;
    auto mark = [&]() {
        if (!timed) return;
        if (!g_stage_ev[stage]) cudaEventCreate(&g_stage_ev[stage]);
        cudaEventRecord(g_stage_ev[stage], stream);
        ++stage;
    };
    int rc;
    mark();
    if ((rc = moe_launch_route(p, stream))) return rc;
    mark();
    if ((rc = moe_launch_dispatch(p, stream))) return rc;
    mark();
    // weight scales -> atoms (independent of the exchange)
    for (int l = 0; l < n_local; ++l) {
        if ((rc = sf_to_atoms_launch(stream, args[l].w1_scale, 0, el * n, k / 32, k / 32, ws[l].w1_atoms))) return rc;
        if ((rc = sf_to_atoms_launch(stream, args[l].w2_scale, 0, el * k, (n / 2) / 32, (n / 2) / 32, ws[l].w2_atoms)))
            return rc;
    }
    mark();
    if ((rc = moe_launch_wait_dispatch(p, stream))) return rc;
    mark();
    for (int l = 0; l < n_local; ++l) {
        const int pe = t->emulated ? l : t->my_pe;
        if ((rc = sf_to_atoms_launch(stream, t->base[pe] + p.lay.recv_scale_off, 0, z.rows_cap, k / 32, z.sld1,
                                     ws[l].recv_atoms)))
            return rc;
    }
    mark();
    if (use_pair) {
        if ((rc = launch_pair_gemm<1, __nv_bfloat16, false>(q1, stream))) return rc;
        mark();
        if ((rc = launch_pair_gemm<2, __nv_bfloat16, false>(q2, stream))) return rc;
    } else {
        if ((rc = launch_gemm<1>(g1, stream))) return rc;
        mark();
        if ((rc = launch_gemm<2>(g2, stream))) return rc;
    }
    mark();
    rc = moe_launch_unpermute(p, stream);
    mark();
    g_stage_count = timed ? stage : 0;
    return rc;
}

// Milliseconds of the stages of the last MoE launch made with debug flag 2 set (after the stream has drained):
// route, quant-dispatch, weight scale atoms, wait for the dispatch, received scale atoms, GEMM1, GEMM2, un-permute.
int moe_stage_ms(float *ms, int capacity) {
    int n = 0;
    for (int i = 0; i + 1 < g_stage_count && n < capacity; ++i, ++n) {
        if (cudaEventElapsedTime(&ms[n], g_stage_ev[i], g_stage_ev[i + 1]) != cudaSuccess) {
            set_error("stage events are not complete (synchronise the stream first)");
            return -1;
        }
    }
    return n;
}

// ------------------------------------------------ standalone all-to-all-v operators ----
struct A2avSizes {
    int rows_cap, sld, nb128;
    size_t counts, recv_codes, recv_scale, combine;                       // symmetric
    size_t idx, eri, meta, recv_atoms, w_atoms;                           // workspace
};

static A2avSizes a2av_sizes(int op, int world, int m, int n, int k, int experts, int fmt = 0) {
    A2avSizes z;
    const int el = experts / world;
    // op 0: a rank can receive every row of every rank; op 1: the rows are already here
    z.rows_cap = static_cast<int>(up(static_cast<size_t>(op == 0 ? world : 1) * m + static_cast<size_t>(el) * 128, 128));
    z.sld = (k / 32 + 1) / 2 * 2;
    z.nb128 = (n + 127) / 128;
    z.counts = up(static_cast<size_t>(world) * experts * 4, 1024);
    z.recv_codes = up(static_cast<size_t>(z.rows_cap) * (fmt ? k / 2 : k), 1024);      // MXFP4: two codes per byte
    z.recv_scale = up(static_cast<size_t>(z.rows_cap) * z.sld, 1024);
    // op 1: a rank gets back one row for every row it contributed, on whichever owner: up to world * m rows
    const size_t out_rows = static_cast<size_t>(op == 1 ? world : 1) * m;
    z.combine = op == 1 ? up(out_rows * n * 2, 1024) : 0;
    z.idx = up(out_rows * 4, 1024);
    z.eri = z.idx;
    z.meta = up(sizeof(MoeMeta), 1024);
    z.recv_atoms = up(sf_atoms_bytes(z.rows_cap, k), 1024);
    z.w_atoms = up(static_cast<size_t>(el) * sf_atoms_bytes(z.nb128 * 128, k), 1024);
    return z;
}

size_t a2av_symmetric_bytes(int op, int world, int m, int n, int k, int experts, int fmt) {
    if (world < 1 || experts < world || experts % world) return 0;
    const A2avSizes z = a2av_sizes(op, world, m, n, k, experts, fmt);
    return z.counts + z.recv_codes + z.recv_scale + z.combine;
}
size_t a2av_workspace_bytes(int op, int world, int m, int n, int k, int experts) {
    if (world < 1 || experts < world || experts % world) return 0;
    const A2avSizes z = a2av_sizes(op, world, m, n, k, experts);
    return z.idx + z.eri + z.meta + z.recv_atoms + z.w_atoms;
}

// weights [E_local][k][n] bytes as a 3-D tensor {n, k, expert}, box {128, 128, 1}: a tile that runs past an
// expert's k rows or n columns is zero-filled
static int encode_b3(const DriverApi *api, CUtensorMap *tm, const void *base, uint64_t n, uint64_t k, uint64_t el) {
    cuuint64_t dims[3] = {n, k, el};
    cuuint64_t strides[2] = {n, n * k};
    cuuint32_t box[3] = {128, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = api->TensorMapEncodeTiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides,
                                           box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (grouped weights) failed: %d", static_cast<int>(r));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

int launch_a2av(int op, int out_dtype, cudaStream_t stream, uint32_t block_num, const A2avArgs *args, void *symmetric,
                int m, int n, int k, int experts, int fmt) {
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
    const int R = t->n_pes;
    if ((op != 0 && op != 1) || (out_dtype != CATCCOS_FP16 && out_dtype != CATCCOS_BF16)) {
        set_error("all-to-all-v grouped matmul: op %d / output type %d not supported (FP16 or BF16)", op, out_dtype);
        return CATCCOS_ERR_INVALID;
    }
    if (m <= 0 || n <= 0 || k <= 0 || (k % 64) != 0 || (n % 16) != 0) {
        set_error("all-to-all-v grouped matmul requires k %% 64 == 0 and n %% 16 == 0 (m=%d n=%d k=%d)", m, n, k);
        return CATCCOS_ERR_INVALID;
    }
    if (fmt != 0 && fmt != 1) {
        set_error("unknown operand format %d (0 = MXFP8, 1 = MXFP4)", fmt);
        return CATCCOS_ERR_INVALID;
    }
    if (fmt == 1 && (k % 256) != 0) {
        set_error("the MXFP4 all-to-all-v operators require k %% 256 == 0 (k=%d)", k);
        return CATCCOS_ERR_INVALID;
    }
    const int kbytes = fmt ? k / 2 : k;      // bytes of one operand row
    if (experts <= 0 || experts % R != 0 || experts > kMoeMaxExperts || experts / R > kMoeMaxLocalExperts) {
        set_error("unsupported expert setup: experts=%d (max %d, divisible by world %d, at most %d per rank)", experts,
                  kMoeMaxExperts, R, kMoeMaxLocalExperts);
        return CATCCOS_ERR_INVALID;
    }
    const int el = experts / R;
    const int n_local = t->emulated ? R : 1;
    const A2avSizes z = a2av_sizes(op, R, m, n, k, experts, fmt);
    const size_t need = z.counts + z.recv_codes + z.recv_scale + z.combine;
    uint8_t *sp = static_cast<uint8_t *>(symmetric);
    uint8_t *hb = t->base[t->my_pe];
    if (sp == nullptr || sp < hb + kFlagBytes || sp + need > hb + t->heap_bytes || ((sp - hb) % 1024) != 0) {
        set_error("symmetric buffer %p (+%zu bytes) is not a 1024-aligned range of the symmetric heap", symmetric, need);
        return CATCCOS_ERR_INVALID;
    }
    const uint64_t off0 = static_cast<uint64_t>(sp - hb);
    int per_rank = t->num_sms / n_local;
    if (block_num > 0 && static_cast<int>(block_num) < per_rank) per_rank = static_cast<int>(block_num);
    if (per_rank < 2) {
        set_error("all-to-all-v grouped matmul needs at least 2 CTAs per rank");
        return CATCCOS_ERR_INVALID;
    }

    MoeParams p;
    memset(&p, 0, sizeof(p));
    p.lay.counts_off = off0;
    p.lay.recv_codes_off = off0 + z.counts;
    p.lay.recv_scale_off = p.lay.recv_codes_off + z.recv_codes;
    p.lay.combine_off = p.lay.recv_scale_off + z.recv_scale;
    p.lay.rows_cap = z.rows_cap;
    p.lay.scale_ld = z.sld;
    for (int pe = 0; pe < R; ++pe) p.heap_base[pe] = t->base[pe];
    p.world = R;
    p.rank_base = t->emulated ? 0 : t->my_pe;
    p.n_local = n_local;
    p.ctas_per_rank = per_rank;
    p.m = op == 1 ? R * m : m;            // rows the routing kernel walks: this rank's row list
    p.K = kbytes;                         // the row-moving kernels count bytes
    p.N = n;
    p.top_k = 1;
    p.experts = experts;
    p.experts_per_rank = el;
    p.epoch = ++t->epoch;
    p.timeout_ns = t->timeout_ns;
    p.status = t->status_dev;

    static thread_local MoePairParams q;
    memset(&q, 0, sizeof(q));
    for (int pe = 0; pe < R; ++pe) q.heap_base[pe] = t->base[pe];
    q.combine_off = p.lay.combine_off;
    q.world = R;
    q.rank_base = p.rank_base;
    q.n_local = n_local;
    q.ctas_per_rank = per_rank & ~1;
    q.rows_cap = z.rows_cap;
    q.experts = experts;
    q.experts_per_rank = el;
    q.epoch = p.epoch;
    q.timeout_ns = p.timeout_ns;
    q.status = p.status;
    q.Kin = kbytes;
    q.fp4 = fmt;
    q.Nw = n;
    q.counter_slot = 2;

    A2avPtrs ptrs;
    memset(&ptrs, 0, sizeof(ptrs));
    ptrs.scale_ld = k / 32;
    uint8_t *w_atoms[kMaxRanks], *recv_atoms[kMaxRanks];
    for (int l = 0; l < n_local; ++l) {
        const A2avArgs &a = args[l];
        if (!a.a || !a.b || !a.c || !a.a_scale || !a.b_scale || !a.local_tokens || !a.workspace ||
            (reinterpret_cast<uintptr_t>(a.a) & 15) || (reinterpret_cast<uintptr_t>(a.b) & 15) ||
            (reinterpret_cast<uintptr_t>(a.c) & 15) || (reinterpret_cast<uintptr_t>(a.workspace) & 255)) {
            set_error("all-to-all-v grouped matmul: every operand must be non-null; tensors 16-byte, workspace 256-byte aligned");
            return CATCCOS_ERR_INVALID;
        }
        uint8_t *w = a.workspace;
        MoeRankArgs &ra = p.ranks[l];
        ra.expert_idx = reinterpret_cast<int *>(w);
        w += z.idx;
        ra.expanded_row_idx = reinterpret_cast<int *>(w);
        w += z.eri;
        ra.meta = reinterpret_cast<MoeMeta *>(w);
        w += z.meta;
        recv_atoms[l] = w;
        w += z.recv_atoms;
        w_atoms[l] = w;
        ra.out = a.c;
        ptrs.codes[l] = a.a;
        ptrs.scales[l] = a.a_scale;
        ptrs.local_tokens[l] = a.local_tokens;
        const int pe = t->emulated ? l : t->my_pe;
        MoePairRankArgs &r = q.ranks[l];
        int rc;
        if ((rc = encode_u8(api, &r.tmA, t->base[pe] + p.lay.recv_codes_off, kbytes, z.rows_cap))) return rc;
        // MXFP8: weights [E_local][k][n] (transB = 0, as the reference's example); MXFP4: K-major [E_local][n][k/2]
        rc = fmt ? encode_u8(api, &r.tmB, a.b, kbytes, static_cast<uint64_t>(el) * n) : encode_b3(api, &r.tmB, a.b, n, k, el);
        if (rc) return rc;
        r.sfa = recv_atoms[l];
        r.sfb = w_atoms[l];
        r.out = a.c;
        r.meta = ra.meta;
    }

    int rc;
    if ((rc = a2av_launch_expert_idx(p, ptrs, stream))) return rc;
    if ((rc = moe_launch_route(p, stream))) return rc;
    if ((rc = a2av_launch_move_rows(p, ptrs, op, stream))) return rc;
    // weight scales [k/64, n, 2] of every local expert -> atoms, each expert padded to whole 128-row atoms
    const size_t expert_atoms = sf_atoms_bytes(z.nb128 * 128, k);
    for (int l = 0; l < n_local; ++l)
        for (int e = 0; e < el; ++e)
            if ((rc = fmt ? sf_to_atoms_launch(stream, args[l].b_scale + static_cast<size_t>(e) * n * (k / 32), 0, n, k / 32, k / 32,
                                               w_atoms[l] + e * expert_atoms)      // [n, k/64, 2] rows of the K-major weights
                          : sf_to_atoms_launch(stream, args[l].b_scale + static_cast<size_t>(e) * (k / 64) * n * 2, 1, n, k / 32, 0,
                                               w_atoms[l] + e * expert_atoms)))
                return rc;
    if (op == 0 && (rc = moe_launch_wait_dispatch(p, stream))) return rc;
    for (int l = 0; l < n_local; ++l) {
        const int pe = t->emulated ? l : t->my_pe;
        if ((rc = sf_to_atoms_launch(stream, t->base[pe] + p.lay.recv_scale_off, 0, z.rows_cap, k / 32, z.sld, recv_atoms[l])))
            return rc;
        {
            // the output has room for world * m rows (as the reference's buffer); rows beyond the real count are zero
            cudaError_t e = cudaMemsetAsync(args[l].c, 0, static_cast<size_t>(R) * m * n * 2, stream);
            if (e != cudaSuccess) {
                set_error("cudaMemsetAsync failed: %s", cudaGetErrorString(e));
                return CATCCOS_ERR_CUDA;
            }
        }
    }
    const bool bf16 = out_dtype == CATCCOS_BF16;
    if (fmt) {      // MXFP4: K-major weights
        if (op == 0)
            return bf16 ? launch_pair_gemm<3, __nv_bfloat16, false>(q, stream) : launch_pair_gemm<3, __half, false>(q, stream);
        rc = bf16 ? launch_pair_gemm<2, __nv_bfloat16, false>(q, stream) : launch_pair_gemm<2, __half, false>(q, stream);
        if (rc) return rc;
        return a2av_launch_copy_out(p, n, stream);
    }
    if (op == 0)
        return bf16 ? launch_pair_gemm<3, __nv_bfloat16, true>(q, stream) : launch_pair_gemm<3, __half, true>(q, stream);
    rc = bf16 ? launch_pair_gemm<2, __nv_bfloat16, true>(q, stream) : launch_pair_gemm<2, __half, true>(q, stream);
    if (rc) return rc;
    return a2av_launch_copy_out(p, n, stream);
}

}  // namespace cb
