// GEMM entry point for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc (or anything that allocates) at the point
// where they need a GEMM: plugins living inside another runtime that owns and budgets all device
// memory (an allocation behind its back breaks its accounting or fails outright), and
// latency-critical loops where an allocation's implicit device synchronisation is not
// acceptable.  The regular launchers need the
// symmetric heap object, which allocates when it is created.  This file offers the single-rank
// tcgen05 GEMM (AllGather-Matmul with a world of one) with the only scratch it needs — the device
// status words and the per-CTA trace slots — in a fixed array that is part of the library image.
#include "../../include/catccos_b200.h"

#include <stdlib.h>

#include <mutex>

#include "dense_ops.h"
#include "gemm_fused.cuh"
#include "ptx.cuh"
#include "symm_heap.h"

using namespace cb;

namespace {

constexpr int kNoAllocMaxCtas = 256;                       // trace slots exist for this many CTAs
constexpr size_t kNoAllocStatusBytes = 256;                // status words, padded
constexpr size_t kNoAllocScratchBytes = kNoAllocStatusBytes + static_cast<size_t>(kNoAllocMaxCtas) * kTraceSlots * 8;
constexpr int kMaxDevices = 64;

// Every GPU that loads the library holds this array (about 33 KiB) until the process exits.
// Host code must never pass `g_no_alloc_scratch` itself to a kernel: on the host the name is only
// a handle for cudaGetSymbolAddress; the device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_no_alloc_scratch[kNoAllocScratchBytes];

struct DeviceSetup {
    bool ready = false;
    unsigned char *scratch = nullptr;   // device address of g_no_alloc_scratch on this device
    int num_sms = 0;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;               // first calls from several host threads set a device up once

template <typename T, bool B_MN>
cudaError_t allow_smem() {
    return cudaFuncSetAttribute(fused_gemm_kernel<OP_AGMM, T, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                kGemmSmemBytes);
}

// Once per device, with that device current: the array's device address and the shared-memory
// attribute of every kernel variant the entry point can launch.
int setup_current_device(DeviceSetup **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("cudaGetDevice failed or device index out of range: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    DeviceSetup &s = g_setup[dev];
    if (!s.ready) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_no_alloc_scratch);      // with `dev` current
        if (e != cudaSuccess || ptr == nullptr) {
            set_error("cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return CATCCOS_ERR_CUDA;
        }
        e = cudaDeviceGetAttribute(&s.num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) e = allow_smem<__nv_bfloat16, true>();
        if (e == cudaSuccess) e = allow_smem<__nv_bfloat16, false>();
        if (e == cudaSuccess) e = allow_smem<__half, true>();
        if (e == cudaSuccess) e = allow_smem<__half, false>();
        if (e != cudaSuccess) {
            set_error("device set-up of the allocation-free GEMM failed: %s", cudaGetErrorString(e));
            return CATCCOS_ERR_CUDA;
        }
        s.scratch = static_cast<unsigned char *>(ptr);
        s.ready = true;
    }
    *out = &s;
    return CATCCOS_OK;
}

// bounded device waits: CATCCOS_WAIT_TIMEOUT_MS as for the other launchers, 10 s by default
uint64_t wait_timeout_ns() {
    if (const char *e = getenv("CATCCOS_WAIT_TIMEOUT_MS")) {
        const long ms = atol(e);
        if (ms > 0) return static_cast<uint64_t>(ms) * 1000000ull;
    }
    return 10ull * 1000 * 1000 * 1000;
}

int encode(const DriverApi *api, CUtensorMap *tm, CUtensorMapDataType dt, const void *base, uint64_t inner,
           uint64_t outer, uint32_t box_inner, uint32_t box_outer) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = api->TensorMapEncodeTiled(tm, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

template <typename T, bool B_MN>
int launch(const FusedParams &p, int grid, cudaStream_t stream) {
    fused_gemm_kernel<OP_AGMM, T, B_MN><<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(p);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("no-alloc GEMM launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

}  // namespace

extern "C" {

int catccos_gemm_no_alloc(void *stream, const void *A, const void *B, void *C, uint32_t m, uint32_t n, uint32_t k,
                          int32_t dataType, uint32_t transB, uint32_t blockNum) {
    DeviceSetup *s = nullptr;
    int rc = setup_current_device(&s);
    if (rc) return rc;
    std::string why;
    const DriverApi *api = driver_api(&why);
    if (!api) {
        set_error("CUDA driver unavailable: %s", why.c_str());
        return CATCCOS_ERR_CUDA;
    }
    if (dataType != CATCCOS_FP16 && dataType != CATCCOS_BF16) {
        set_error("catccos_gemm_no_alloc takes FP16 (1) or BF16 (27), got %d", dataType);
        return CATCCOS_ERR_INVALID;
    }
    if (!A || !B || !C || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
        (reinterpret_cast<uintptr_t>(C) & 15)) {
        set_error("A, B and C must be non-null and 16-byte aligned");
        return CATCCOS_ERR_INVALID;
    }
    if (m == 0 || n == 0 || k == 0 || (k % 8) != 0 || (n % 8) != 0 || m > (1u << 30) || n > (1u << 30) ||
        k > (1u << 30)) {
        set_error("unsupported shape m=%u n=%u k=%u (n and k multiples of 8, each dimension at most 2^30)", m, n, k);
        return CATCCOS_ERR_INVALID;
    }
    int grid = s->num_sms;
    if (blockNum > 0 && static_cast<int>(blockNum) < grid) grid = static_cast<int>(blockNum);
    if (grid > kNoAllocMaxCtas) {
        set_error("grid of %d CTAs exceeds the %d CTAs the built-in scratch array has slots for; pass blockNum <= %d",
                  grid, kNoAllocMaxCtas, kNoAllocMaxCtas);
        return CATCCOS_ERR_INVALID;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // the array keeps the previous call's contents: status words and trace slots start from zero
    cudaError_t e = cudaMemsetAsync(s->scratch, 0, kNoAllocScratchBytes, st);
    if (e != cudaSuccess) {
        set_error("cudaMemsetAsync failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    FusedParams p;
    memset(&p, 0, sizeof(p));
    const CUtensorMapDataType dt =
        dataType == CATCCOS_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    RankArgs &ra = p.ranks[0];
    if ((rc = encode(api, &ra.tmA, dt, A, k, m, BK, BM))) return rc;
    rc = transB ? encode(api, &ra.tmB, dt, B, k, n, BK, BN) : encode(api, &ra.tmB, dt, B, n, k, 64, BK);
    if (rc) return rc;
    ra.tmAg = ra.tmA;
    ra.A = A;
    ra.C = C;
    p.world = 1;
    p.rank_base = 0;
    p.n_local = 1;
    p.ctas_per_rank = grid;
    p.push_ctas = 0;
    p.M = static_cast<int>(m);
    p.N = static_cast<int>(n);
    p.K = static_cast<int>(k);
    p.epoch = 1;
    p.compute_only = 0;
    p.timeout_ns = wait_timeout_ns();
    p.status = reinterpret_cast<int *>(s->scratch);
    p.trace = reinterpret_cast<unsigned long long *>(s->scratch + kNoAllocStatusBytes);
    const bool bf16 = dataType == CATCCOS_BF16;
    if (bf16) return transB ? launch<__nv_bfloat16, false>(p, grid, st) : launch<__nv_bfloat16, true>(p, grid, st);
    return transB ? launch<__half, false>(p, grid, st) : launch<__half, true>(p, grid, st);
}

int catccos_gemm_no_alloc_status(int32_t *words8, uint64_t *trace, uint32_t traceCtas) {
    DeviceSetup *s = nullptr;
    int rc = setup_current_device(&s);
    if (rc) return rc;
    if (traceCtas > static_cast<uint32_t>(kNoAllocMaxCtas)) {
        set_error("traceCtas %u exceeds %d", traceCtas, kNoAllocMaxCtas);
        return CATCCOS_ERR_INVALID;
    }
    cudaError_t e = cudaDeviceSynchronize();
    int w[ST_WORDS] = {0};
    if (e == cudaSuccess) e = cudaMemcpy(w, s->scratch, sizeof(w), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && trace && traceCtas)
        e = cudaMemcpy(trace, s->scratch + kNoAllocStatusBytes, static_cast<size_t>(traceCtas) * kTraceSlots * 8,
                       cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        set_error("reading the scratch array failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    if (words8)
        for (int i = 0; i < ST_WORDS; ++i) words8[i] = w[i];
    if (w[ST_CODE] != 0) {
        set_error("device wait ran out: code=%d site=%d", w[ST_CODE], w[ST_WHERE]);
        return CATCCOS_ERR_DEVICE_WAIT;
    }
    return CATCCOS_OK;
}

}  // extern "C"
