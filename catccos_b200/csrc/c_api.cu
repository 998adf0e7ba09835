// extern "C" surface (include/catccos_b200.h).
#include "../../include/catccos_b200.h"

#include "dense_ops.h"
#include "fp4_gemm.h"
#include "moe_ops.h"
#include "mx_ops.h"
#include "mx_quant.h"
#include "mxq_allgather.h"
#include "ptx.cuh"
#include "sched.h"
#include "symm_heap.h"

#include <algorithm>

using namespace cb;

namespace {

__global__ void wait_unset_flag_kernel(const uint32_t *flag, uint32_t expected, uint64_t timeout_ns, int *status) {
    __shared__ int abort_flag;
    abort_flag = 0;
    WaitCtl ctl;
    ctl.abort_smem = &abort_flag;
    ctl.status = status;
    ctl.deadline_ns = globaltimer_ns() + timeout_ns;
    ctl.rank = 0;
    wait_flag_ge(flag, expected, ctl, W_TEST, 0);
}

int dense_op_of(int32_t commType) {
    switch (commType) {
        case CATCCOS_MATMUL_ALLREDUCE: return OP_MMAR;
        case CATCCOS_ALLGATHER_MATMUL:
        case CATCCOS_ASCEND950_ALLGATHER_MATMUL:
        case CATCCOS_ALLGATHER_MATMUL_WITH_GATHER_RESULT:
        case CATCCOS_ALLGATHER_MATMUL_REMOTE_READ:
        case CATCCOS_ASCEND950_ALLTOALL_MATMUL: return OP_AGMM;
        case CATCCOS_MATMUL_REDUCE_SCATTER:
        case CATCCOS_ASCEND950_MATMUL_REDUCE_SCATTER: return OP_MMRS;
        case CATCCOS_ASCEND950_MATMUL_ALLTOALL: return OP_MMA2A;
        default: return -1;
    }
}

// all-to-all-v grouped matmul family: returns 1 and sets op (0 dispatch-GMM, 1 GMM-combine) and fmt (0 MXFP8, 1 MXFP4)
int a2av_kind_of(int32_t commType, int *op, int *fmt) {
    switch (commType) {
        case CATCCOS_ASCEND950_FP8_MX_ALLTOALLV_GROUPED_MATMUL: *op = 0; *fmt = 0; return 1;
        case CATCCOS_ASCEND950_FP8_MX_GROUPED_MATMUL_ALLTOALLV: *op = 1; *fmt = 0; return 1;
        case CATCCOS_ASCEND950_FP4_MX_ALLTOALLV_GROUPED_MATMUL: *op = 0; *fmt = 1; return 1;
        case CATCCOS_ASCEND950_FP4_MX_GROUPED_MATMUL_ALLTOALLV: *op = 1; *fmt = 1; return 1;
        default: return 0;
    }
}

int dense_flow_of(int32_t commType) {
    return commType == CATCCOS_ALLGATHER_MATMUL_WITH_GATHER_RESULT ? 1
           : commType == CATCCOS_ALLGATHER_MATMUL_REMOTE_READ      ? 2
           : commType == CATCCOS_ASCEND950_ALLTOALL_MATMUL         ? 3
                                                                    : 0;
}

int check_tiling(const CocTilingParams *tiling) {
    Team *t = team();
    if (!t) {
        set_error("symmetric heap not initialised (call catccos_shmem_init first)");
        return CATCCOS_ERR_NOT_INIT;
    }
    if (!tiling) {
        set_error("tiling is NULL");
        return CATCCOS_ERR_INVALID;
    }
    if (tiling->rankSize != 0 && static_cast<int>(tiling->rankSize) != t->n_pes) {
        set_error("tiling.rankSize (%u) differs from the number of PEs (%d)", tiling->rankSize, t->n_pes);
        return CATCCOS_ERR_INVALID;
    }
    return CATCCOS_OK;
}

// `flow`: 0 = the operator as such; 1 = AllGather-Matmul that also returns the gathered A in customPtrs[0]
// (examples/allgather_matmul_with_gather_result/allgather_matmul_with_gather_result_host.h:54); 2 = remote-read
// AllGather-Matmul (examples/allgather_matmul_remote_read); 3 = AllToAll-Matmul (examples/ascend950_alltoall_matmul:
// tiling.m = rows of every rank's A, block d of which goes to rank d).
int launch_dense_abi(int op, int dtype, void *stream, uint32_t blockNum, CatccosKernelParams *params, int n_params,
                     uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA, uint32_t transB, int flow = 0) {
    int rc = check_tiling(tiling);
    if (rc) return rc;
    if (!params) {
        set_error("params is NULL");
        return CATCCOS_ERR_INVALID;
    }
    Team *t = team();
    const int want = t->emulated ? t->n_pes : 1;
    if (n_params != want) {
        set_error(t->emulated ? "emulated PEs: use catccos_launch_emulated with one parameter block per PE"
                              : "catccos_launch_emulated needs catccos_shmem_init_emulated");
        return CATCCOS_ERR_INVALID;
    }
    DenseArgs args[kMaxRanks];
    for (int i = 0; i < n_params; ++i) {
        args[i] = {params[i].ptrA, params[i].ptrB, params[i].ptrC};
        if (flow == 1) {
            if (params[i].customCount < 1 || !params[i].customPtrs || !params[i].customPtrs[0]) {
                set_error("AllGatherMatmulWithGatherResult expects customPtrs = {gatherA [rankSize*m, k]}");
                return CATCCOS_ERR_INVALID;
            }
            args[i].gather_out = params[i].customPtrs[0];
        }
    }
    int m = static_cast<int>(tiling->m);
    if (flow == 3) {
        if (m % t->n_pes != 0) {
            set_error("AllToAll-Matmul needs m (%d) divisible by the world size (%d)", m, t->n_pes);
            return CATCCOS_ERR_INVALID;
        }
        m /= t->n_pes;
    }
    return launch_dense(op, dtype, static_cast<cudaStream_t>(stream), blockNum, args, symmetric, m,
                        static_cast<int>(tiling->n), static_cast<int>(tiling->k), static_cast<int>(transA),
                        static_cast<int>(transB), flow == 2 ? AG_REMOTE_READ : flow == 3 ? AG_ALLTOALL : AG_PUSH);
}

int launch_mx_ag_abi(int dtype, void *stream, uint32_t blockNum, CatccosKernelParams *params, int n_params,
                     uint8_t **workspaces, uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA,
                     uint32_t transB, int fmt = 0) {
    int rc = check_tiling(tiling);
    if (rc) return rc;
    Team *t = team();
    const int want = t->emulated ? t->n_pes : 1;
    if (!params || n_params != want || !workspaces) {
        set_error("MXFP8 AllGather-Matmul: one parameter block and one workspace per local PE are required");
        return CATCCOS_ERR_INVALID;
    }
    if (transA) {
        set_error("transA=1 is not supported");
        return CATCCOS_ERR_INVALID;
    }
    MxAgArgs args[kMaxRanks];
    for (int i = 0; i < n_params; ++i) {
        if (params[i].customCount < 2 || !params[i].customPtrs) {
            set_error("MXFP8 AllGather-Matmul expects customPtrs = {aScale, bScale}");
            return CATCCOS_ERR_INVALID;
        }
        args[i] = {params[i].ptrA, params[i].ptrB, params[i].ptrC, params[i].customPtrs[0], params[i].customPtrs[1],
                   workspaces[i]};
    }
    return launch_mx_allgather_matmul(dtype, static_cast<cudaStream_t>(stream), blockNum, args, symmetric,
                                      static_cast<int>(tiling->m), static_cast<int>(tiling->n),
                                      static_cast<int>(tiling->k), static_cast<int>(transB), fmt);
}

// MXFP8 Matmul-ReduceScatter: KernelParams as set by the example's operator class
// (examples/ascend950_mxfp8_matmul_reduce_scatter/ascend950_mxfp8_matmul_reduce_scatter_host.h:107:
// SetKernelParams(a, b, c, aScale, bScale)).
int launch_mx_rs_abi(int dtype, int code_format, void *stream, uint32_t blockNum, CatccosKernelParams *params,
                     int n_params, uint8_t **workspaces, uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA,
                     uint32_t transB, int alltoall = 0) {
    int rc = check_tiling(tiling);
    if (rc) return rc;
    Team *t = team();
    const int want = t->emulated ? t->n_pes : 1;
    if (!params || n_params != want || !workspaces) {
        set_error("MXFP8 Matmul-ReduceScatter: one parameter block and one workspace per local PE are required");
        return CATCCOS_ERR_INVALID;
    }
    if (transA) {
        set_error("transA=1 is not supported");
        return CATCCOS_ERR_INVALID;
    }
    MxAgArgs args[kMaxRanks];
    for (int i = 0; i < n_params; ++i) {
        if (params[i].customCount < 2 || !params[i].customPtrs) {
            set_error("MXFP8 Matmul-ReduceScatter expects customPtrs = {aScale, bScale}");
            return CATCCOS_ERR_INVALID;
        }
        args[i] = {params[i].ptrA, params[i].ptrB, params[i].ptrC, params[i].customPtrs[0], params[i].customPtrs[1],
                   workspaces[i]};
    }
    return launch_mx_matmul_reduce_scatter(dtype, code_format, static_cast<cudaStream_t>(stream), blockNum, args,
                                           symmetric, static_cast<int>(tiling->m), static_cast<int>(tiling->n),
                                           static_cast<int>(tiling->k), static_cast<int>(transB), alltoall);
}

int launch_moe_abi(void *stream, uint32_t blockNum, CatccosKernelParams *params, int n_params, uint8_t **workspaces,
                   uint8_t *symmetric, CocTilingParams *tiling) {
    int rc = check_tiling(tiling);
    if (rc) return rc;
    Team *t = team();
    const int want = t->emulated ? t->n_pes : 1;
    if (!params || n_params != want || !workspaces) {
        set_error("dispatch_ffn_combine: one parameter block and one workspace per local PE are required");
        return CATCCOS_ERR_INVALID;
    }
    if (tiling->epSize != 0 && static_cast<int>(tiling->epSize) != t->n_pes) {
        set_error("tiling.epSize (%u) must equal the number of PEs (%d)", tiling->epSize, t->n_pes);
        return CATCCOS_ERR_INVALID;
    }
    MoeArgs args[kMaxRanks];
    for (int i = 0; i < n_params; ++i) {
        if (params[i].customCount < 5 || !params[i].customPtrs) {
            set_error("dispatch_ffn_combine expects customPtrs = {b2, expertIdx, probs, bScale, b2Scale}");
            return CATCCOS_ERR_INVALID;
        }
        uint8_t **c = params[i].customPtrs;
        args[i] = {params[i].ptrA, params[i].ptrB, params[i].ptrC, c[0], reinterpret_cast<const int *>(c[1]),
                   reinterpret_cast<const float *>(c[2]), c[3], c[4], workspaces[i]};
    }
    return launch_moe_dispatch_ffn_combine(static_cast<cudaStream_t>(stream), blockNum, args, symmetric,
                                           static_cast<int>(tiling->m), static_cast<int>(tiling->k),
                                           static_cast<int>(tiling->n), static_cast<int>(tiling->topK),
                                           static_cast<int>(tiling->expertNum));
}

// Standalone MXFP8 AllToAllV-GroupedMatmul (op 0) / GroupedMatmul-AllToAllV (op 1): KernelParams as set by the
// examples' operator classes (examples/ascend950_fp8_mx_alltoallv_grouped_matmul/..._host.h:118):
// SetKernelParams(a, b, c, aScale, bScale, localTokensPerExpert, globalTokensPerLocalExpert).
int launch_a2av_abi(int op, int dtype, void *stream, uint32_t blockNum, CatccosKernelParams *params, int n_params,
                    uint8_t **workspaces, uint8_t *symmetric, CocTilingParams *tiling, int fmt = 0) {
    int rc = check_tiling(tiling);
    if (rc) return rc;
    Team *t = team();
    const int want = t->emulated ? t->n_pes : 1;
    if (!params || n_params != want || !workspaces) {
        set_error("all-to-all-v grouped matmul: one parameter block and one workspace per local PE are required");
        return CATCCOS_ERR_INVALID;
    }
    if (tiling->epSize != 0 && static_cast<int>(tiling->epSize) != t->n_pes) {
        set_error("tiling.epSize (%u) must equal the number of PEs (%d): tensor-parallel groups inside an expert group are "
                  "not supported", tiling->epSize, t->n_pes);
        return CATCCOS_ERR_INVALID;
    }
    A2avArgs args[kMaxRanks];
    for (int i = 0; i < n_params; ++i) {
        if (params[i].customCount < 3 || !params[i].customPtrs) {
            set_error("all-to-all-v grouped matmul expects customPtrs = {aScale, bScale, localTokensPerExpert, "
                      "globalTokensPerLocalExpert}");
            return CATCCOS_ERR_INVALID;
        }
        uint8_t **c = params[i].customPtrs;
        args[i] = {params[i].ptrA, params[i].ptrB, params[i].ptrC, c[0], c[1], reinterpret_cast<const int *>(c[2]),
                   workspaces[i]};
    }
    return launch_a2av(op, dtype, static_cast<cudaStream_t>(stream), blockNum, args, symmetric, static_cast<int>(tiling->m),
                       static_cast<int>(tiling->n), static_cast<int>(tiling->k), static_cast<int>(tiling->expertNum), fmt);
}

int launch_mxq_ag_abi(void *stream, uint32_t blockNum, CatccosKernelParams *params, int n_params, uint8_t *symmetric,
                      CocTilingParams *tiling) {
    int rc = check_tiling(tiling);
    if (rc) return rc;
    Team *t = team();
    const int want = t->emulated ? t->n_pes : 1;
    if (!params || n_params != want) {
        set_error("MX quant + AllGather: one parameter block per local PE is required");
        return CATCCOS_ERR_INVALID;
    }
    MxqAgArgs args[kMaxRanks];
    for (int i = 0; i < n_params; ++i) args[i] = {params[i].ptrA, params[i].ptrC, params[i].ptrB};
    return launch_mx_quant_allgather(static_cast<cudaStream_t>(stream), blockNum, args, symmetric,
                                     static_cast<int>(tiling->m), static_cast<int>(tiling->n));
}

}  // namespace

int catccos_mx_quant(void *stream, const void *inputBf16, uint8_t *codes, uint8_t *scales, uint8_t *sfAtoms,
                     uint32_t rows, uint32_t k) {
    const int nb = static_cast<int>(k / 32);
    return mx_quant_launch(static_cast<cudaStream_t>(stream), inputBf16, static_cast<int>(rows), static_cast<int>(k),
                           codes, k, scales, (nb + 1) / 2 * 2, sfAtoms);
}
size_t catccos_sf_atoms_bytes(uint32_t rows, uint32_t k) { return sf_atoms_bytes(static_cast<int>(rows), static_cast<int>(k)); }

// ---- host-buffer form ------------------------------------------------------------------
namespace {
constexpr int kHostRunChunks = 8;
struct HostRunCache {
    void *dA = nullptr, *dB = nullptr, *dC = nullptr;
    size_t bytesA = 0, bytesB = 0, bytesC = 0;
    const void *b_host = nullptr;                                // dense operators: the host buffer a resident B came from
    size_t b_bytes = 0;
    void *b_dev = nullptr;
    cudaStream_t in = nullptr, run = nullptr, out = nullptr;     // host->device, kernels, device->host
    cudaEvent_t landed[kHostRunChunks + 1] = {};                  // B, then every chunk of A
    cudaEvent_t done[kHostRunChunks] = {};                        // a chunk's rows of C are complete
    bool ready = false;
    // operands of the block-scaled and MoE operators: device copy, its capacity, and what it holds
    struct Operand {
        void *dev = nullptr;
        size_t cap = 0;
        const void *host = nullptr;      // host buffer a resident copy came from
        size_t bytes = 0;
    } opnd[3 + 8], work;
} g_hr;

int ensure(void **p, size_t *have, size_t want) {
    if (*have >= want && *p) return CATCCOS_OK;
    if (*p) cudaFree(*p);
    *p = nullptr;
    *have = 0;
    cudaError_t e = cudaMalloc(p, want);
    if (e != cudaSuccess) {
        set_error("cudaMalloc(%zu) failed: %s", want, cudaGetErrorString(e));
        return CATCCOS_ERR_NOMEM;
    }
    *have = want;
    return CATCCOS_OK;
}
int ensure_host_run_streams() {
    if (g_hr.ready) return CATCCOS_OK;
    cudaError_t e = cudaStreamCreateWithFlags(&g_hr.in, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&g_hr.run, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&g_hr.out, cudaStreamNonBlocking);
    for (int i = 0; i <= kHostRunChunks && e == cudaSuccess; ++i)
        e = cudaEventCreateWithFlags(&g_hr.landed[i], cudaEventDisableTiming);
    for (int i = 0; i < kHostRunChunks && e == cudaSuccess; ++i)
        e = cudaEventCreateWithFlags(&g_hr.done[i], cudaEventDisableTiming);
    if (e != cudaSuccess) {
        set_error("creating the host-buffer path's streams failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    g_hr.ready = true;
    return CATCCOS_OK;
}
void release_host_run_cache() {
    if (g_hr.dA) cudaFree(g_hr.dA);
    if (g_hr.dB) cudaFree(g_hr.dB);
    if (g_hr.dC) cudaFree(g_hr.dC);
    for (auto &o : g_hr.opnd)
        if (o.dev) cudaFree(o.dev);
    if (g_hr.work.dev) cudaFree(g_hr.work.dev);
    if (g_hr.in) cudaStreamDestroy(g_hr.in);
    if (g_hr.run) cudaStreamDestroy(g_hr.run);
    if (g_hr.out) cudaStreamDestroy(g_hr.out);
    for (cudaEvent_t ev : g_hr.landed)
        if (ev) cudaEventDestroy(ev);
    for (cudaEvent_t ev : g_hr.done)
        if (ev) cudaEventDestroy(ev);
    g_hr = HostRunCache();
}
// after the streams have drained: a bounded device wait that ran out must not pass for success
int host_run_status() {
    int w[ST_WORDS];
    int rc = team_read_status(w);
    if (rc) return rc;
    if (w[ST_CODE] == ERR_PARTIAL_RANGE) {
        set_error("rank %d sent a partial product beyond the fp16 range of the reduce-scatter exchange: the result is not "
                  "valid; set CATCCOS_RS_EXCHANGE=native to exchange partials in the output type", w[ST_RANK]);
        return CATCCOS_ERR_RANGE;
    }
    if (w[ST_CODE] != 0) {
        set_error("device wait ran out: code=%d site=%d rank=%d index=%d expected=%d seen=%d", w[ST_CODE], w[ST_WHERE],
                  w[ST_RANK], w[ST_INDEX], w[ST_EXPECTED], w[ST_SEEN]);
        return CATCCOS_ERR_DEVICE_WAIT;
    }
    return CATCCOS_OK;
}
}  // namespace


extern "C" {

int catccos_shmem_init(int32_t my_pe, int32_t n_pes, uint64_t local_mem_size, const char *ip_port) {
    return team_init(my_pe, n_pes, local_mem_size, ip_port);
}
int catccos_shmem_init_emulated(int32_t n_pes, uint64_t local_mem_size) {
    return team_init_emulated(n_pes, local_mem_size);
}
int catccos_shmem_finalize(void) {
    release_host_run_cache();
    return team_finalize();
}
void *catccos_shmem_malloc(size_t bytes) { return team_malloc(bytes); }
void catccos_shmem_free(void *ptr) {
    if (ptr) team_free(ptr);
}
void *catccos_shmem_ptr(const void *ptr, int32_t pe) { return team_ptr(ptr, pe); }
int catccos_shmem_get_host(void *hostDst, const void *ptr, int32_t pe, size_t bytes) {
    void *src = team_ptr(ptr, pe);
    if (!src || !hostDst) {
        set_error("catccos_shmem_get_host: bad pointer or PE");
        return CATCCOS_ERR_INVALID;
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(hostDst, src, bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        set_error("catccos_shmem_get_host failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}
int catccos_shmem_put_host(void *ptr, int32_t pe, const void *hostSrc, size_t bytes) {
    void *dst = team_ptr(ptr, pe);
    if (!dst || !hostSrc) {
        set_error("catccos_shmem_put_host: bad pointer or PE");
        return CATCCOS_ERR_INVALID;
    }
    cudaError_t e = cudaMemcpy(dst, hostSrc, bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        set_error("catccos_shmem_put_host failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}
int32_t catccos_shmem_my_pe(void) { return team() ? team()->my_pe : -1; }
int32_t catccos_shmem_n_pes(void) { return team() ? team()->n_pes : 0; }
int catccos_shmem_barrier_all(void) {
    if (!team()) {
        set_error("symmetric heap not initialised");
        return CATCCOS_ERR_NOT_INIT;
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        set_error("cudaDeviceSynchronize failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return team_host_barrier();
}

const char *catccos_last_error(void) { return last_error(); }

int catccos_last_status(int32_t *words8) {
    if (!team()) {
        set_error("symmetric heap not initialised");
        return CATCCOS_ERR_NOT_INIT;
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        set_error("cudaDeviceSynchronize failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    int w[ST_WORDS];
    int rc = team_read_status(w);
    if (rc) return rc;
    if (words8)
        for (int i = 0; i < ST_WORDS; ++i) words8[i] = w[i];
    if (w[ST_CODE] == ERR_PARTIAL_RANGE) {
        set_error("rank %d sent a partial product beyond the fp16 range of the reduce-scatter exchange: the result is not "
                  "valid; set CATCCOS_RS_EXCHANGE=native to exchange partials in the output type", w[ST_RANK]);
        return CATCCOS_ERR_RANGE;
    }
    if (w[ST_CODE] != 0) {
        set_error("device wait ran out: code=%d site=%d rank=%d index=%d expected=%d seen=%d", w[ST_CODE], w[ST_WHERE],
                  w[ST_RANK], w[ST_INDEX], w[ST_EXPECTED], w[ST_SEEN]);
        return CATCCOS_ERR_DEVICE_WAIT;
    }
    return CATCCOS_OK;
}
int catccos_reset_status(void) { return team_reset_status(); }

int catccos_debug_wait_unset_flag(void *stream, uint32_t timeout_ms) {
    Team *t = team();
    if (!t) {
        set_error("symmetric heap not initialised");
        return CATCCOS_ERR_NOT_INIT;
    }
    // the last word of the flag region is never written by any operator
    const uint32_t *flag = reinterpret_cast<const uint32_t *>(t->base[t->my_pe]) + (kFlagWords - 1);
    wait_unset_flag_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
        flag, 0x7fffffffu, static_cast<uint64_t>(timeout_ms) * 1000000ull, t->status_dev);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

int catccos_debug_set_flags(uint32_t flags) {
    if (!team()) {
        set_error("symmetric heap not initialised");
        return CATCCOS_ERR_NOT_INIT;
    }
    team()->debug_flags = flags;
    return CATCCOS_OK;
}

int catccos_debug_moe_stage_ms(float *ms, int32_t capacity) {
    if (!ms || capacity < 1) {
        set_error("catccos_debug_moe_stage_ms: bad arguments");
        return -1;
    }
    return moe_stage_ms(ms, capacity);
}

int catccos_debug_set_trace(void *device_buf) {
    if (!team()) {
        set_error("symmetric heap not initialised");
        return CATCCOS_ERR_NOT_INIT;
    }
    team()->trace_dev = static_cast<unsigned long long *>(device_buf);
    return CATCCOS_OK;
}

int catccos_debug_rs_tile_order(int32_t world, int32_t rank, int32_t rows_per_rank, int32_t n, int32_t pairs, int32_t *out,
                                int32_t capacity, int32_t *lag) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || rows_per_rank < 1 || n < 1 || pairs < 1 ||
        (!out && capacity > 0)) {
        set_error("catccos_debug_rs_tile_order: invalid argument");
        return -CATCCOS_ERR_INVALID;
    }
    const int nt = (n + BN - 1) / BN, stripes = (rows_per_rank + 2 * BM - 1) / (2 * BM);
    const RsOrder o = rs_order_make(world, nt, stripes, pairs);
    if (lag) *lag = o.lag;
    const int tiles = rs_order_tiles(o);
    for (int t = 0; t < tiles && t < capacity; ++t) rs_order_decode(o, rank, t, out[3 * t], out[3 * t + 1], out[3 * t + 2]);
    return tiles;
}

int catccos_debug_ag_tile_order(int32_t world, int32_t rank, int32_t m, int32_t n, int32_t group, int32_t *out,
                                int32_t capacity) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || m < 1 || n < 1 || (!out && capacity > 0)) {
        set_error("catccos_debug_ag_tile_order: invalid argument");
        return -CATCCOS_ERR_INVALID;
    }
    const int nt = (n + BN - 1) / BN, mt2 = (m + 2 * BM - 1) / (2 * BM);
    const int tiles = world * mt2 * nt;
    if (group < 1) group = 1;
    for (int t = 0; t < tiles && t < capacity; ++t)
        ag_order_grouped(world, mt2, nt, group, rank, t, out[3 * t], out[3 * t + 1], out[3 * t + 2]);
    return tiles;
}

int catccos_debug_ag_group_rows(int64_t tile_bytes, int32_t pairs, int64_t l2_budget_bytes) {
    if (tile_bytes < 1 || pairs < 1 || l2_budget_bytes < 1) {
        set_error("catccos_debug_ag_group_rows: invalid argument");
        return -CATCCOS_ERR_INVALID;
    }
    return ag_order_group_rows(tile_bytes, pairs, l2_budget_bytes);
}

int catccos_debug_ag_push_order(int32_t world, int32_t rank, int32_t m, int32_t *out, int32_t capacity) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || m < 1 || (!out && capacity > 0)) {
        set_error("catccos_debug_ag_push_order: invalid argument");
        return -CATCCOS_ERR_INVALID;
    }
    const int units_per_dest = ((m + BM - 1) / BM) * kAgSubChunks;
    const int total = (world - 1) * units_per_dest;
    for (int u = 0; u < total && u < capacity; ++u) {
        int d, cu;
        ag_push_decode(world, units_per_dest, rank, u, d, cu);
        out[3 * u] = d;
        out[3 * u + 1] = cu / kAgSubChunks;
        out[3 * u + 2] = cu % kAgSubChunks;
    }
    return total;
}

int catccos_debug_slot_sequence(const uint64_t *sigs, const uint8_t *foreign_before, int32_t n, int32_t *half,
                                int32_t *need_back) {
    if (!sigs || !half || !need_back || n < 0) {
        set_error("catccos_debug_slot_sequence: invalid argument");
        return CATCCOS_ERR_INVALID;
    }
    Team t;     // a scratch team: only its launch bookkeeping is used
    for (int i = 0; i < n; ++i) {
        if (foreign_before && foreign_before[i]) ++t.epoch;
        const uint32_t epoch = t.epoch + 1;
        const LaunchSlot s = peek_slot(&t, sigs[i], epoch);
        commit_slot(&t, sigs[i], epoch, s);
        half[i] = s.half;
        need_back[i] = static_cast<int32_t>(epoch - s.entered_need);
    }
    return CATCCOS_OK;
}

size_t catccos_fp4_gemm_workspace_bytes(int32_t format, uint32_t m, uint32_t n, uint32_t k) {
    return fp4_gemm_workspace_bytes(format, static_cast<int>(m), static_cast<int>(n), static_cast<int>(k));
}
int catccos_fp4_gemm(void *stream, int32_t format, int32_t dataType, const void *A, const void *B, void *C, const void *aScale,
                     const void *bScale, float alpha, uint32_t m, uint32_t n, uint32_t k, void *workspace, uint32_t blockNum) {
    if (m > (1u << 30) || n > (1u << 30) || k > (1u << 30)) {
        set_error("catccos_fp4_gemm: dimension too large");
        return CATCCOS_ERR_INVALID;
    }
    return launch_fp4_gemm(static_cast<cudaStream_t>(stream), format, dataType, static_cast<const uint8_t *>(A),
                           static_cast<const uint8_t *>(B), C, static_cast<const uint8_t *>(aScale),
                           static_cast<const uint8_t *>(bScale), alpha, static_cast<int>(m), static_cast<int>(n),
                           static_cast<int>(k), static_cast<uint8_t *>(workspace), blockNum);
}

size_t catccos_symmetric_bytes(int32_t commType, int32_t dataType, const CocTilingParams *tiling) {
    (void)dataType;
    if (!tiling) return 0;
    const int world = tiling->rankSize ? static_cast<int>(tiling->rankSize) : (team() ? team()->n_pes : 1);
    const int op = dense_op_of(commType);
    if (op >= 0)
        return dense_symmetric_bytes(op, world, static_cast<int>(tiling->m) / (dense_flow_of(commType) == 3 ? world : 1),
                                     static_cast<int>(tiling->n), static_cast<int>(tiling->k));
    if (commType == CATCCOS_ASCEND950_FP8_MX_ALLGATHER_MATMUL || commType == CATCCOS_ASCEND950_FP4_MX_ALLGATHER_MATMUL)
        return mx_ag_symmetric_bytes(world, static_cast<int>(tiling->m), static_cast<int>(tiling->n),
                                     static_cast<int>(tiling->k), commType == CATCCOS_ASCEND950_FP4_MX_ALLGATHER_MATMUL ? 1 : 0);
    if (commType == CATCCOS_ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER || commType == CATCCOS_ASCEND950_MXFP8_MATMUL_ALLTOALL ||
        commType == CATCCOS_ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER)
        return dense_symmetric_bytes(OP_MMRS, world, static_cast<int>(tiling->m), static_cast<int>(tiling->n),
                                     static_cast<int>(tiling->k));
    if (commType == CATCCOS_MX_QUANT_ALLGATHER)
        return mxq_allgather_symmetric_bytes(world, static_cast<int>(tiling->m), static_cast<int>(tiling->n));
    int a2_op = 0, a2_fmt = 0;
    if (a2av_kind_of(commType, &a2_op, &a2_fmt) && tiling->expertNum > 0)
        return a2av_symmetric_bytes(a2_op, world, static_cast<int>(tiling->m), static_cast<int>(tiling->n),
                                    static_cast<int>(tiling->k), static_cast<int>(tiling->expertNum), a2_fmt);
    if (commType == CATCCOS_ASCEND950_DISPATCH_FFN_COMBINE && tiling->expertNum > 0)
        return moe_symmetric_bytes(world, static_cast<int>(tiling->m), static_cast<int>(tiling->k),
                                   static_cast<int>(tiling->n), static_cast<int>(tiling->topK),
                                   static_cast<int>(tiling->expertNum));
    return 0;
}
size_t catccos_workspace_bytes(int32_t commType, int32_t dataType, const CocTilingParams *tiling) {
    (void)dataType;
    if (tiling && (commType == CATCCOS_ASCEND950_FP8_MX_ALLGATHER_MATMUL || commType == CATCCOS_ASCEND950_FP4_MX_ALLGATHER_MATMUL ||
                   commType == CATCCOS_ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER ||
                   commType == CATCCOS_ASCEND950_MXFP8_MATMUL_ALLTOALL ||
                   commType == CATCCOS_ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER))
        return mx_ag_workspace_bytes(static_cast<int>(tiling->m), static_cast<int>(tiling->n),
                                     static_cast<int>(tiling->k));
    int a2_op = 0, a2_fmt = 0;
    if (tiling && a2av_kind_of(commType, &a2_op, &a2_fmt) && tiling->expertNum > 0) {
        const int world = tiling->rankSize ? static_cast<int>(tiling->rankSize) : (team() ? team()->n_pes : 1);
        return a2av_workspace_bytes(a2_op, world,
                                    static_cast<int>(tiling->m), static_cast<int>(tiling->n), static_cast<int>(tiling->k),
                                    static_cast<int>(tiling->expertNum));
    }
    if (tiling && commType == CATCCOS_ASCEND950_DISPATCH_FFN_COMBINE && tiling->expertNum > 0) {
        const int world = tiling->rankSize ? static_cast<int>(tiling->rankSize) : (team() ? team()->n_pes : 1);
        return moe_workspace_bytes(world, static_cast<int>(tiling->m), static_cast<int>(tiling->k),
                                   static_cast<int>(tiling->n), static_cast<int>(tiling->topK),
                                   static_cast<int>(tiling->expertNum));
    }
    return 0;   // the dense operators keep everything in the symmetric region
}

#define DENSE_LAUNCH(name, op, dtype)                                                                          \
    int name(void *stream, uint32_t blockNum, uint64_t fftsAddr, CatccosKernelParams *params, uint8_t *workspace, \
             uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA, uint32_t transB) {                    \
        (void)fftsAddr;                                                                                          \
        (void)workspace;                                                                                         \
        return launch_dense_abi(op, dtype, stream, blockNum, params, 1, symmetric, tiling, transA, transB);      \
    }
#define DENSE_FLOW_LAUNCH(name, flow, dtype)                                                                     \
    int name(void *stream, uint32_t blockNum, uint64_t fftsAddr, CatccosKernelParams *params, uint8_t *workspace, \
             uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA, uint32_t transB) {                    \
        (void)fftsAddr;                                                                                          \
        (void)workspace;                                                                                         \
        return launch_dense_abi(OP_AGMM, dtype, stream, blockNum, params, 1, symmetric, tiling, transA, transB, flow); \
    }
DENSE_FLOW_LAUNCH(LaunchAllGatherMatmulWithGatherResultFP16, 1, CATCCOS_FP16)
DENSE_FLOW_LAUNCH(LaunchAllGatherMatmulWithGatherResultBF16, 1, CATCCOS_BF16)
DENSE_FLOW_LAUNCH(LaunchAllGatherMatmulRemoteReadFP16, 2, CATCCOS_FP16)
DENSE_FLOW_LAUNCH(LaunchAllGatherMatmulRemoteReadBF16, 2, CATCCOS_BF16)
DENSE_FLOW_LAUNCH(LaunchAscend950AllToAllMatmulFP16, 3, CATCCOS_FP16)
DENSE_FLOW_LAUNCH(LaunchAscend950AllToAllMatmulBF16, 3, CATCCOS_BF16)
DENSE_LAUNCH(LaunchAscend950MatmulAllToAllFP16, OP_MMA2A, CATCCOS_FP16)
DENSE_LAUNCH(LaunchAscend950MatmulAllToAllBF16, OP_MMA2A, CATCCOS_BF16)
DENSE_LAUNCH(LaunchMatmulAllReduceFP16, OP_MMAR, CATCCOS_FP16)
DENSE_LAUNCH(LaunchMatmulAllReduceBF16, OP_MMAR, CATCCOS_BF16)
DENSE_LAUNCH(LaunchAllGatherMatmulFP16, OP_AGMM, CATCCOS_FP16)
DENSE_LAUNCH(LaunchAllGatherMatmulBF16, OP_AGMM, CATCCOS_BF16)
DENSE_LAUNCH(LaunchMatmulReduceScatterFP16, OP_MMRS, CATCCOS_FP16)
DENSE_LAUNCH(LaunchMatmulReduceScatterBF16, OP_MMRS, CATCCOS_BF16)
DENSE_LAUNCH(LaunchAscend950AllGatherMatmulFP16, OP_AGMM, CATCCOS_FP16)
DENSE_LAUNCH(LaunchAscend950AllGatherMatmulBF16, OP_AGMM, CATCCOS_BF16)
DENSE_LAUNCH(LaunchAscend950MatmulReduceScatterFP16, OP_MMRS, CATCCOS_FP16)
DENSE_LAUNCH(LaunchAscend950MatmulReduceScatterBF16, OP_MMRS, CATCCOS_BF16)

#define MXAG_LAUNCH(name, dtype, fmt)                                                                          \
    int name(void *stream, uint32_t blockNum, uint64_t fftsAddr, CatccosKernelParams *params, uint8_t *workspace, \
             uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA, uint32_t transB) {                    \
        (void)fftsAddr;                                                                                          \
        return launch_mx_ag_abi(dtype, stream, blockNum, params, 1, &workspace, symmetric, tiling, transA, transB, fmt); \
    }
MXAG_LAUNCH(LaunchAscend950Fp8MxAllGatherMatmulFP16, CATCCOS_FP16, 0)
MXAG_LAUNCH(LaunchAscend950Fp8MxAllGatherMatmulBF16, CATCCOS_BF16, 0)
MXAG_LAUNCH(LaunchAscend950Fp4MxAllGatherMatmulFP16, CATCCOS_FP16, 1)
MXAG_LAUNCH(LaunchAscend950Fp4MxAllGatherMatmulBF16, CATCCOS_BF16, 1)

#define MXRS_LAUNCH(name, dtype, fmt)                                                                          \
    int name(void *stream, uint32_t blockNum, uint64_t fftsAddr, CatccosKernelParams *params, uint8_t *workspace, \
             uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA, uint32_t transB) {                    \
        (void)fftsAddr;                                                                                          \
        return launch_mx_rs_abi(dtype, fmt, stream, blockNum, params, 1, &workspace, symmetric, tiling, transA, transB); \
    }
#define MXA2A_LAUNCH(name, dtype)                                                                              \
    int name(void *stream, uint32_t blockNum, uint64_t fftsAddr, CatccosKernelParams *params, uint8_t *workspace, \
             uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA, uint32_t transB) {                    \
        (void)fftsAddr;                                                                                          \
        return launch_mx_rs_abi(dtype, 0, stream, blockNum, params, 1, &workspace, symmetric, tiling, transA, transB, 1); \
    }
MXA2A_LAUNCH(LaunchAscend950MxFp8MatmulAllToAllFP16, CATCCOS_FP16)
MXA2A_LAUNCH(LaunchAscend950MxFp8MatmulAllToAllBF16, CATCCOS_BF16)
MXRS_LAUNCH(LaunchAscend950Fp4MxMatmulReduceScatterFP16, CATCCOS_FP16, 2)
MXRS_LAUNCH(LaunchAscend950Fp4MxMatmulReduceScatterBF16, CATCCOS_BF16, 2)
MXRS_LAUNCH(LaunchAscend950MxFp8MatmulReduceScatterFP16, CATCCOS_FP16, 1)
MXRS_LAUNCH(LaunchAscend950MxFp8MatmulReduceScatterBF16, CATCCOS_BF16, 1)
MXRS_LAUNCH(LaunchAscend950MxFp8E4M3MatmulReduceScatterFP16, CATCCOS_FP16, 0)
MXRS_LAUNCH(LaunchAscend950MxFp8E4M3MatmulReduceScatterBF16, CATCCOS_BF16, 0)

#define A2AV_LAUNCH(name, op, dtype) A2AV_LAUNCH_F(name, op, dtype, 0)
#define A2AV_LAUNCH_F(name, op, dtype, fmt)                                                                    \
    int name(void *stream, uint32_t blockNum, uint64_t fftsAddr, CatccosKernelParams *params, uint8_t *workspace, \
             uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA, uint32_t transB) {                    \
        (void)fftsAddr;                                                                                          \
        (void)transA;                                                                                            \
        (void)transB;                                                                                            \
        return launch_a2av_abi(op, dtype, stream, blockNum, params, 1, &workspace, symmetric, tiling, fmt);      \
    }
A2AV_LAUNCH_F(LaunchAscend950Fp4MxAllToAllVGroupedMatmulFP16, 0, CATCCOS_FP16, 1)
A2AV_LAUNCH_F(LaunchAscend950Fp4MxAllToAllVGroupedMatmulBF16, 0, CATCCOS_BF16, 1)
A2AV_LAUNCH_F(LaunchAscend950Fp4MxGroupedMatmulAllToAllVFP16, 1, CATCCOS_FP16, 1)
A2AV_LAUNCH_F(LaunchAscend950Fp4MxGroupedMatmulAllToAllVBF16, 1, CATCCOS_BF16, 1)
A2AV_LAUNCH(LaunchAscend950Fp8MxAllToAllVGroupedMatmulFP16, 0, CATCCOS_FP16)
A2AV_LAUNCH(LaunchAscend950Fp8MxAllToAllVGroupedMatmulBF16, 0, CATCCOS_BF16)
A2AV_LAUNCH(LaunchAscend950Fp8MxGroupedMatmulAllToAllVFP16, 1, CATCCOS_FP16)
A2AV_LAUNCH(LaunchAscend950Fp8MxGroupedMatmulAllToAllVBF16, 1, CATCCOS_BF16)

int LaunchAscend950BF16QuantAllGatherFP8E4M3FN(void *stream, uint32_t blockNum, uint64_t fftsAddr, CatccosKernelParams *params,
                                               uint8_t *workspace, uint8_t *symmetric, CocTilingParams *tiling,
                                               uint32_t transA, uint32_t transB) {
    (void)fftsAddr;
    (void)workspace;
    (void)transA;
    (void)transB;
    return launch_mxq_ag_abi(stream, blockNum, params, 1, symmetric, tiling);
}

int LaunchAscend950DispatchFFNCombineBF16(void *stream, uint32_t blockNum, uint64_t fftsAddr, CatccosKernelParams *params,
                                          uint8_t *workspace, uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA,
                                          uint32_t transB) {
    (void)fftsAddr;
    (void)transA;
    (void)transB;
    return launch_moe_abi(stream, blockNum, params, 1, &workspace, symmetric, tiling);
}

int catccos_launch(int32_t commType, int32_t dataType, void *stream, uint32_t blockNum, uint64_t fftsAddr,
                   CatccosKernelParams *params, uint8_t *workspace, uint8_t *symmetric, CocTilingParams *tiling,
                   uint32_t transA, uint32_t transB) {
    (void)fftsAddr;
    const int op = dense_op_of(commType);
    if (op >= 0 && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_dense_abi(op, dataType, stream, blockNum, params, 1, symmetric, tiling, transA, transB,
                                dense_flow_of(commType));
    if (commType == CATCCOS_ASCEND950_FP8_MX_ALLGATHER_MATMUL && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_mx_ag_abi(dataType, stream, blockNum, params, 1, &workspace, symmetric, tiling, transA, transB);
    if (commType == CATCCOS_ASCEND950_FP4_MX_ALLGATHER_MATMUL && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_mx_ag_abi(dataType, stream, blockNum, params, 1, &workspace, symmetric, tiling, transA, transB, 1);
    if (commType == CATCCOS_ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_mx_rs_abi(dataType, 1, stream, blockNum, params, 1, &workspace, symmetric, tiling, transA, transB);
    if (commType == CATCCOS_ASCEND950_MXFP8_MATMUL_ALLTOALL && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_mx_rs_abi(dataType, 0, stream, blockNum, params, 1, &workspace, symmetric, tiling, transA, transB, 1);
    if (commType == CATCCOS_ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_mx_rs_abi(dataType, 2, stream, blockNum, params, 1, &workspace, symmetric, tiling, transA, transB);
    if (commType == CATCCOS_ASCEND950_DISPATCH_FFN_COMBINE && dataType == CATCCOS_BF16)
        return launch_moe_abi(stream, blockNum, params, 1, &workspace, symmetric, tiling);
    if (commType == CATCCOS_MX_QUANT_ALLGATHER && dataType == CATCCOS_FP8E4M3FN)
        return launch_mxq_ag_abi(stream, blockNum, params, 1, symmetric, tiling);
    int a2_op = 0, a2_fmt = 0;
    if (a2av_kind_of(commType, &a2_op, &a2_fmt) && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_a2av_abi(a2_op, dataType, stream, blockNum, params, 1, &workspace, symmetric, tiling, a2_fmt);
    set_error("no kernel registered for commType=%d dataType=%d", commType, dataType);
    return CATCCOS_ERR_INVALID;
}

int catccos_launch_emulated(int32_t commType, int32_t dataType, void *stream, uint32_t blockNum,
                            CatccosKernelParams *params, uint8_t **workspaces, uint8_t *symmetric,
                            CocTilingParams *tiling, uint32_t transA, uint32_t transB) {
    Team *t = team();
    if (!t || !t->emulated) {
        set_error("catccos_launch_emulated needs catccos_shmem_init_emulated");
        return t ? CATCCOS_ERR_INVALID : CATCCOS_ERR_NOT_INIT;
    }
    const int op = dense_op_of(commType);
    if (op >= 0 && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_dense_abi(op, dataType, stream, blockNum, params, t->n_pes, symmetric, tiling, transA, transB,
                                dense_flow_of(commType));
    if (commType == CATCCOS_ASCEND950_FP8_MX_ALLGATHER_MATMUL && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_mx_ag_abi(dataType, stream, blockNum, params, t->n_pes, workspaces, symmetric, tiling, transA,
                                transB);
    if (commType == CATCCOS_ASCEND950_FP4_MX_ALLGATHER_MATMUL && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_mx_ag_abi(dataType, stream, blockNum, params, t->n_pes, workspaces, symmetric, tiling, transA,
                                transB, 1);
    if (commType == CATCCOS_ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_mx_rs_abi(dataType, 1, stream, blockNum, params, t->n_pes, workspaces, symmetric, tiling, transA,
                                transB);
    if (commType == CATCCOS_ASCEND950_MXFP8_MATMUL_ALLTOALL && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_mx_rs_abi(dataType, 0, stream, blockNum, params, t->n_pes, workspaces, symmetric, tiling, transA,
                                transB, 1);
    if (commType == CATCCOS_ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_mx_rs_abi(dataType, 2, stream, blockNum, params, t->n_pes, workspaces, symmetric, tiling, transA,
                                transB);
    if (commType == CATCCOS_ASCEND950_DISPATCH_FFN_COMBINE && dataType == CATCCOS_BF16)
        return launch_moe_abi(stream, blockNum, params, t->n_pes, workspaces, symmetric, tiling);
    if (commType == CATCCOS_MX_QUANT_ALLGATHER && dataType == CATCCOS_FP8E4M3FN)
        return launch_mxq_ag_abi(stream, blockNum, params, t->n_pes, symmetric, tiling);
    int a2_op = 0, a2_fmt = 0;
    if (a2av_kind_of(commType, &a2_op, &a2_fmt) && (dataType == CATCCOS_FP16 || dataType == CATCCOS_BF16))
        return launch_a2av_abi(a2_op, dataType, stream, blockNum, params, t->n_pes, workspaces, symmetric, tiling, a2_fmt);
    set_error("no kernel registered for commType=%d dataType=%d", commType, dataType);
    return CATCCOS_ERR_INVALID;
}

// Operand sizes (bytes) of the operators the host-buffer form serves beyond the dense ones; slot 0/1/2 = A/B/C,
// 3.. = customPtrs in the operator's order.  Returns the number of custom operands, or -1.
static int host_operand_bytes(int32_t commType, const CocTilingParams *t, size_t R, size_t *bytes) {
    const size_t m = t->m, n = t->n, k = t->k;
    if (commType == CATCCOS_ASCEND950_FP8_MX_ALLGATHER_MATMUL || commType == CATCCOS_ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER) {
        const bool ag = commType == CATCCOS_ASCEND950_FP8_MX_ALLGATHER_MATMUL;
        bytes[0] = m * k;
        bytes[1] = k * n;
        bytes[2] = (ag ? R * m : m / R) * n * 2;
        bytes[3] = m * (k / 64) * 2;
        bytes[4] = (k / 64) * n * 2;
        return 2;
    }
    if (commType == CATCCOS_ASCEND950_DISPATCH_FFN_COMBINE && t->expertNum > 0 && t->topK > 0) {
        const size_t el = t->expertNum / R, tk = t->topK;
        bytes[0] = m * k * 2;
        bytes[1] = el * n * k;
        bytes[2] = m * k * 2;
        bytes[3] = el * k * (n / 2);
        bytes[4] = m * tk * 4;
        bytes[5] = m * tk * 4;
        bytes[6] = el * n * (k / 32);
        bytes[7] = el * k * (n / 64);
        return 5;
    }
    return -1;
}

static int run_host_general(int32_t commType, int32_t dataType, uint32_t blockNum, const void *hostA, const void *hostB,
                            void *hostC, const void *const *hostCustom, uint32_t customCount, CocTilingParams *tiling,
                            uint32_t transA, uint32_t transB, uint32_t residentMask) {
    Team *t = team();
    const size_t R = t->n_pes;
    size_t bytes[3 + 8] = {};
    const int nc = host_operand_bytes(commType, tiling, R, bytes);
    if (nc < 0) {
        set_error("catccos_run_host: no host-buffer path for commType=%d dataType=%d", commType, dataType);
        return CATCCOS_ERR_INVALID;
    }
    if (!hostA || !hostB || !hostC || customCount < static_cast<uint32_t>(nc) || !hostCustom) {
        set_error("host buffers must not be NULL (this operator takes %d custom operands)", nc);
        return CATCCOS_ERR_INVALID;
    }
    int rc = ensure_host_run_streams();
    if (rc) return rc;
    const void *src[3 + 8] = {hostA, hostB, nullptr};
    for (int i = 0; i < nc; ++i) {
        if (!hostCustom[i]) {
            set_error("custom host buffer %d is NULL", i);
            return CATCCOS_ERR_INVALID;
        }
        src[3 + i] = hostCustom[i];
    }
    // inputs: a resident operand (bit i of the mask; bit 0 = A, 1 = B, 3.. = custom) is copied when its host buffer
    // or size is new, every other input on every call
    for (int i = 0; i < 3 + nc; ++i) {
        auto &o = g_hr.opnd[i];
        if ((rc = ensure(&o.dev, &o.cap, std::max<size_t>(bytes[i], 256)))) return rc;
        if (i == 2) continue;
        const bool resident = (residentMask >> i) & 1u;
        if (resident && o.host == src[i] && o.bytes == bytes[i]) continue;
        cudaMemcpyAsync(o.dev, src[i], bytes[i], cudaMemcpyHostToDevice, g_hr.run);
        o.host = resident ? src[i] : nullptr;
        o.bytes = bytes[i];
    }
    const size_t wbytes = catccos_workspace_bytes(commType, dataType, tiling);
    if (wbytes > g_hr.work.cap) {
        if ((rc = ensure(&g_hr.work.dev, &g_hr.work.cap, wbytes))) return rc;
        cudaMemsetAsync(g_hr.work.dev, 0, wbytes, g_hr.run);
    }
    CocTilingParams til = *tiling;
    til.rankSize = static_cast<uint32_t>(R);
    const size_t need = catccos_symmetric_bytes(commType, dataType, &til);
    void *symm = nullptr;
    if (need > 0 && !(symm = team_top_region(need))) return CATCCOS_ERR_NOMEM;
    uint8_t *custom[8];
    for (int i = 0; i < nc; ++i) custom[i] = static_cast<uint8_t *>(g_hr.opnd[3 + i].dev);
    CatccosKernelParams kp{static_cast<uint8_t *>(g_hr.opnd[0].dev), static_cast<uint8_t *>(g_hr.opnd[1].dev),
                           static_cast<uint8_t *>(g_hr.opnd[2].dev), custom, static_cast<uint32_t>(nc)};
    rc = catccos_launch(commType, dataType, g_hr.run, blockNum, 0, &kp, static_cast<uint8_t *>(g_hr.work.dev),
                        static_cast<uint8_t *>(symm), tiling, transA, transB);
    if (!rc) cudaMemcpyAsync(hostC, g_hr.opnd[2].dev, bytes[2], cudaMemcpyDeviceToHost, g_hr.run);
    cudaError_t e = cudaStreamSynchronize(g_hr.run);
    if (e != cudaSuccess) {
        set_error("host-buffer run failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    if (rc) return rc;
    return host_run_status();
}

int catccos_run_host_resident(int32_t commType, int32_t dataType, uint32_t blockNum, const void *hostA, const void *hostB,
                              void *hostC, const void *const *hostCustom, uint32_t customCount, CocTilingParams *tiling,
                              uint32_t transA, uint32_t transB, uint32_t residentMask);

static int run_host_any(int32_t commType, int32_t dataType, uint32_t blockNum, const void *hostA, const void *hostB,
                        void *hostC, const void *const *hostCustom, uint32_t customCount, CocTilingParams *tiling,
                        uint32_t transA, uint32_t transB, uint32_t residentMask) {
    int rc = check_tiling(tiling);
    if (rc) return rc;
    Team *t = team();
    if (t->emulated) {
        set_error("catccos_run_host needs one process per PE (catccos_shmem_init)");
        return CATCCOS_ERR_INVALID;
    }
    const int op = dense_op_of(commType);
    if (op < 0)
        return run_host_general(commType, dataType, blockNum, hostA, hostB, hostC, hostCustom, customCount, tiling, transA,
                                transB, residentMask);
    if (dense_flow_of(commType) != 0 || op == OP_MMA2A) {
        set_error("catccos_run_host: no host-buffer path for commType=%d (the data-flow variants take device buffers)", commType);
        return CATCCOS_ERR_INVALID;
    }
    if (residentMask & ~2u) {
        set_error("catccos_run_host_resident: of the dense operators' operands only B (bit 1) can stay resident");
        return CATCCOS_ERR_INVALID;
    }
    if (dataType != CATCCOS_FP16 && dataType != CATCCOS_BF16) {
        set_error("catccos_run_host: no host-buffer path for commType=%d dataType=%d", commType, dataType);
        return CATCCOS_ERR_INVALID;
    }
    if (!hostA || !hostB || !hostC) {
        set_error("host buffers must not be NULL");
        return CATCCOS_ERR_INVALID;
    }
    const size_t m = tiling->m, n = tiling->n, k = tiling->k, R = t->n_pes;
    const size_t bytesA = m * k * 2, bytesB = k * n * 2;
    const size_t bytesC = (op == OP_AGMM ? R * m : op == OP_MMRS ? m / R : m) * n * 2;
    const size_t need = dense_symmetric_bytes(op, static_cast<int>(R), static_cast<int>(m), static_cast<int>(n),
                                              static_cast<int>(k));
    if ((rc = ensure(&g_hr.dA, &g_hr.bytesA, bytesA)) || (rc = ensure(&g_hr.dB, &g_hr.bytesB, bytesB)) ||
        (rc = ensure(&g_hr.dC, &g_hr.bytesC, bytesC)) || (rc = ensure_host_run_streams()))
        return rc;
    // a resident B is copied when its host buffer, size or device copy is new
    const bool copy_b = !((residentMask & 2u) && g_hr.b_host == hostB && g_hr.b_bytes == bytesB && g_hr.b_dev == g_hr.dB);
    g_hr.b_host = (residentMask & 2u) ? hostB : nullptr;
    g_hr.b_bytes = bytesB;
    g_hr.b_dev = g_hr.dB;
    // the symmetric region of this path sits at the end of the heap, outside the stack that the
    // caller's catccos_shmem_malloc / catccos_shmem_free calls grow and shrink
    void *symm = nullptr;
    if (need > 0 && !(symm = team_top_region(need))) return CATCCOS_ERR_NOMEM;
    cudaError_t e = cudaSuccess;
    if (R == 1 && m >= 2 * 256 * kHostRunChunks) {
        // One PE: the operator is a plain GEMM, so it is cut into row chunks and the three stages
        // overlap -- chunk i's rows of C travel to the host while chunk i+1 is multiplied and chunk
        // i+2 is still arriving.  B goes first (every chunk needs all of it).
        const size_t rows_per = (m / kHostRunChunks + 255) / 256 * 256;
        if (copy_b) cudaMemcpyAsync(g_hr.dB, hostB, bytesB, cudaMemcpyHostToDevice, g_hr.in);
        cudaEventRecord(g_hr.landed[0], g_hr.in);
        cudaStreamWaitEvent(g_hr.run, g_hr.landed[0], 0);
        int chunk = 0;
        for (size_t r0 = 0; r0 < m && !rc; r0 += rows_per, ++chunk) {
            const size_t rows = std::min(rows_per, m - r0);
            uint8_t *a = static_cast<uint8_t *>(g_hr.dA) + r0 * k * 2;
            uint8_t *c = static_cast<uint8_t *>(g_hr.dC) + r0 * n * 2;
            cudaMemcpyAsync(a, static_cast<const uint8_t *>(hostA) + r0 * k * 2, rows * k * 2, cudaMemcpyHostToDevice, g_hr.in);
            cudaEventRecord(g_hr.landed[chunk + 1], g_hr.in);
            cudaStreamWaitEvent(g_hr.run, g_hr.landed[chunk + 1], 0);
            CocTilingParams sub = *tiling;
            sub.m = static_cast<uint32_t>(rows);
            CatccosKernelParams kp{a, static_cast<uint8_t *>(g_hr.dB), c, nullptr, 0};
            rc = launch_dense_abi(op, dataType, g_hr.run, blockNum, &kp, 1, nullptr, &sub, transA, transB);
            if (rc) break;
            cudaEventRecord(g_hr.done[chunk], g_hr.run);
            cudaStreamWaitEvent(g_hr.out, g_hr.done[chunk], 0);
            cudaMemcpyAsync(static_cast<uint8_t *>(hostC) + r0 * n * 2, c, rows * n * 2, cudaMemcpyDeviceToHost, g_hr.out);
        }
        e = cudaStreamSynchronize(g_hr.in);
        if (e == cudaSuccess) e = cudaStreamSynchronize(g_hr.run);
        if (e == cudaSuccess) e = cudaStreamSynchronize(g_hr.out);
    } else {
        // several PEs: the fused launch needs this rank's whole A and B; the copies are stream-ordered around it
        cudaMemcpyAsync(g_hr.dA, hostA, bytesA, cudaMemcpyHostToDevice, g_hr.run);
        if (copy_b) cudaMemcpyAsync(g_hr.dB, hostB, bytesB, cudaMemcpyHostToDevice, g_hr.run);
        CatccosKernelParams kp{static_cast<uint8_t *>(g_hr.dA), static_cast<uint8_t *>(g_hr.dB),
                               static_cast<uint8_t *>(g_hr.dC), nullptr, 0};
        rc = launch_dense_abi(op, dataType, g_hr.run, blockNum, &kp, 1, static_cast<uint8_t *>(symm), tiling, transA,
                              transB);
        if (!rc) cudaMemcpyAsync(hostC, g_hr.dC, bytesC, cudaMemcpyDeviceToHost, g_hr.run);
        e = cudaStreamSynchronize(g_hr.run);
    }
    if (e != cudaSuccess) {
        set_error("host-buffer run failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    if (rc) return rc;
    return host_run_status();
}

int catccos_run_host(int32_t commType, int32_t dataType, uint32_t blockNum, const void *hostA, const void *hostB,
                     void *hostC, const void *const *hostCustom, uint32_t customCount, CocTilingParams *tiling,
                     uint32_t transA, uint32_t transB) {
    return run_host_any(commType, dataType, blockNum, hostA, hostB, hostC, hostCustom, customCount, tiling, transA, transB, 0);
}

int catccos_run_host_resident(int32_t commType, int32_t dataType, uint32_t blockNum, const void *hostA, const void *hostB,
                              void *hostC, const void *const *hostCustom, uint32_t customCount, CocTilingParams *tiling,
                              uint32_t transA, uint32_t transB, uint32_t residentMask) {
    return run_host_any(commType, dataType, blockNum, hostA, hostB, hostC, hostCustom, customCount, tiling, transA, transB,
                        residentMask);
}

}  // extern "C"
