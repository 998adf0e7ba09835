// Operator identifiers and parameter blocks of the host-side operator layer; same names, values
// and field order as the reference's utils/info.h (enums :46-93, CocTilingParams :95-114,
// KernelParams :123-167, FreeDeviceSpace :169-193, name maps :196-275).
#ifndef CATCCOS_HOST_INFO_H
#define CATCCOS_HOST_INFO_H

#include <cstdint>
#include <map>
#include <string>

#include "../catccos_b200.h"
#include "utils.h"

constexpr uint32_t M0 = 128;                 // tcgen05 tile of the dense kernels (the reference: 128 x 256 x 256)
constexpr uint32_t N0 = 256;
constexpr uint32_t K0 = 64;
constexpr uint32_t WARM_UP_TIMES = 10;
constexpr uint32_t PERF_TEST_CYCLE_TIMES = 3;
constexpr uint64_t SHMEM_MALLOC_MAX_SIZE = 1024UL * 1024UL * 1024;
constexpr uint64_t SHMEM_BUFF_BYTES = 1004UL * 1024 * 1024;
constexpr int32_t MAX_RANK_SIZE = 8;

enum CocCommType {
    MATMUL_ALLREDUCE = CATCCOS_MATMUL_ALLREDUCE,
    ALLGATHER_MATMUL = CATCCOS_ALLGATHER_MATMUL,
    ASCEND950_ALLGATHER_MATMUL = CATCCOS_ASCEND950_ALLGATHER_MATMUL,
    MATMUL_REDUCE_SCATTER = CATCCOS_MATMUL_REDUCE_SCATTER,
    ASCEND950_MATMUL_REDUCE_SCATTER = CATCCOS_ASCEND950_MATMUL_REDUCE_SCATTER,
    ALLGATHER_MATMUL_WITH_GATHER_RESULT = CATCCOS_ALLGATHER_MATMUL_WITH_GATHER_RESULT,
    ALLGATHER_MATMUL_REMOTE_READ = CATCCOS_ALLGATHER_MATMUL_REMOTE_READ,
    ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER = CATCCOS_ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER,
    ASCEND950_MXFP8_MATMUL_ALLTOALL = CATCCOS_ASCEND950_MXFP8_MATMUL_ALLTOALL,
    ASCEND950_FP8_MX_ALLGATHER_MATMUL = CATCCOS_ASCEND950_FP8_MX_ALLGATHER_MATMUL,
    ASCEND950_FP4_MX_ALLGATHER_MATMUL = CATCCOS_ASCEND950_FP4_MX_ALLGATHER_MATMUL,
    MX_QUANT_ALLGATHER = CATCCOS_MX_QUANT_ALLGATHER,
    ASCEND950_FP8_MX_GROUPED_MATMUL_ALLTOALLV = CATCCOS_ASCEND950_FP8_MX_GROUPED_MATMUL_ALLTOALLV,
    ASCEND950_FP8_MX_ALLTOALLV_GROUPED_MATMUL = CATCCOS_ASCEND950_FP8_MX_ALLTOALLV_GROUPED_MATMUL,
    ASCEND950_FP4_MX_GROUPED_MATMUL_ALLTOALLV = CATCCOS_ASCEND950_FP4_MX_GROUPED_MATMUL_ALLTOALLV,
    ASCEND950_FP4_MX_ALLTOALLV_GROUPED_MATMUL = CATCCOS_ASCEND950_FP4_MX_ALLTOALLV_GROUPED_MATMUL,
    ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER = CATCCOS_ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER,
    ASCEND950_DISPATCH_FFN_COMBINE = CATCCOS_ASCEND950_DISPATCH_FFN_COMBINE,
    UNKNOWN = 36,
    ASCEND950_ALLTOALL_MATMUL = CATCCOS_ASCEND950_ALLTOALL_MATMUL,     // no counterparts in the reference's enum
    ASCEND950_MATMUL_ALLTOALL = CATCCOS_ASCEND950_MATMUL_ALLTOALL
};

enum CocDataType { FP16 = CATCCOS_FP16, INT8 = CATCCOS_INT8, BF16 = CATCCOS_BF16, FP8E4M3FN = CATCCOS_FP8E4M3FN };

// CocTilingParams is the C struct of the C-ABI (17 uint32 fields, reference order).

// Owns the custom pointer array like the reference's KernelParams; device buffers are released
// with FreeDeviceSpace().
struct KernelParams : CatccosKernelParams {
    KernelParams() : CatccosKernelParams{nullptr, nullptr, nullptr, nullptr, 0} {}
    KernelParams(const KernelParams &) = delete;
    KernelParams &operator=(const KernelParams &) = delete;

    template <typename... Args>
    void SetKernelParams(uint8_t *a, uint8_t *b, uint8_t *c, Args... args) {
        ptrA = a;
        ptrB = b;
        ptrC = c;
        delete[] customPtrs;
        customPtrs = nullptr;
        customCount = sizeof...(args);
        if (customCount > 0) {
            uint8_t *ptrs[] = {args..., nullptr};
            customPtrs = new uint8_t *[customCount];
            for (uint32_t i = 0; i < customCount; ++i) customPtrs[i] = ptrs[i];
        }
    }
    ~KernelParams() { delete[] customPtrs; }
};

inline void FreeDeviceSpace(KernelParams &params) {
    if (params.ptrA) CUDA_CHECK(cudaFree(params.ptrA));
    if (params.ptrB) CUDA_CHECK(cudaFree(params.ptrB));
    if (params.ptrC) CUDA_CHECK(cudaFree(params.ptrC));
    params.ptrA = params.ptrB = params.ptrC = nullptr;
    for (uint32_t i = 0; i < params.customCount; ++i)
        if (params.customPtrs[i]) {
            CUDA_CHECK(cudaFree(params.customPtrs[i]));
            params.customPtrs[i] = nullptr;
        }
}

// short CLI names (utils/info.h:196-230)
inline const std::map<std::string, CocCommType> &CommTypeMap() {
    static const std::map<std::string, CocCommType> m = {
        {"mmar", MATMUL_ALLREDUCE},
        {"agmm", ALLGATHER_MATMUL},
        {"a5agmm", ASCEND950_ALLGATHER_MATMUL},
        {"mmrs", MATMUL_REDUCE_SCATTER},
        {"a5mmrs", ASCEND950_MATMUL_REDUCE_SCATTER},
        {"agmmwg", ALLGATHER_MATMUL_WITH_GATHER_RESULT},
        {"agmmrr", ALLGATHER_MATMUL_REMOTE_READ},
        {"a5atamm", ASCEND950_ALLTOALL_MATMUL},
        {"a5mmata", ASCEND950_MATMUL_ALLTOALL},
        {"a5fp8mxagmm", ASCEND950_FP8_MX_ALLGATHER_MATMUL},
        {"a5fp4mxagmm", ASCEND950_FP4_MX_ALLGATHER_MATMUL},
        {"a5fp4mmrs", ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER},
        {"a5mxfp8mmrs", ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER},
        {"a5mxfp8mmata", ASCEND950_MXFP8_MATMUL_ALLTOALL},
        {"a5moe", ASCEND950_DISPATCH_FFN_COMBINE},
        {"mxqtag", MX_QUANT_ALLGATHER},
        {"a5fp8gmmata", ASCEND950_FP8_MX_GROUPED_MATMUL_ALLTOALLV},
        {"a5fp8mxatavgmm", ASCEND950_FP8_MX_ALLTOALLV_GROUPED_MATMUL},
        {"a5fp4gmmata", ASCEND950_FP4_MX_GROUPED_MATMUL_ALLTOALLV},
        {"a5fp4mxatavgmm", ASCEND950_FP4_MX_ALLTOALLV_GROUPED_MATMUL},
    };
    return m;
}
inline CocCommType GetCommType(const std::string &kernelName) {
    const auto it = CommTypeMap().find(kernelName);
    return it == CommTypeMap().end() ? UNKNOWN : it->second;
}
// registered operator names (utils/info.h:242-275)
inline const std::map<CocCommType, std::string> &CommTypeOpNameMap() {
    static const std::map<CocCommType, std::string> m = {
        {MATMUL_ALLREDUCE, "MatmulAllReduce"},
        {ALLGATHER_MATMUL, "AllGatherMatmul"},
        {ASCEND950_ALLGATHER_MATMUL, "Ascend950AllGatherMatmul"},
        {MATMUL_REDUCE_SCATTER, "MatmulReduceScatter"},
        {ASCEND950_MATMUL_REDUCE_SCATTER, "Ascend950MatmulReduceScatter"},
        {ALLGATHER_MATMUL_WITH_GATHER_RESULT, "AllGatherMatmulWithGatherResult"},
        {ALLGATHER_MATMUL_REMOTE_READ, "AllGatherMatmulRemoteRead"},
        {ASCEND950_ALLTOALL_MATMUL, "Ascend950AllToAllMatmul"},
        {ASCEND950_MATMUL_ALLTOALL, "Ascend950MatmulAllToAll"},
        {ASCEND950_FP8_MX_ALLGATHER_MATMUL, "Ascend950Fp8MxAllGatherMatmul"},
        {ASCEND950_FP4_MX_ALLGATHER_MATMUL, "Ascend950Fp4MxAllGatherMatmul"},
        {ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER, "Ascend950Fp4MxMatmulReduceScatter"},
        {ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER, "Ascend950MxFp8MatmulReduceScatter"},
        {ASCEND950_MXFP8_MATMUL_ALLTOALL, "Ascend950MxFp8MatmulAllToAll"},
        {ASCEND950_DISPATCH_FFN_COMBINE, "Ascend950DispatchFFNCombine"},
        {MX_QUANT_ALLGATHER, "MxQuantAllGather"},
        {ASCEND950_FP8_MX_GROUPED_MATMUL_ALLTOALLV, "Ascend950Fp8MxGroupedMatmulAllToAllV"},
        {ASCEND950_FP8_MX_ALLTOALLV_GROUPED_MATMUL, "Ascend950Fp8MxAllToAllVGroupedMatmul"},
        {ASCEND950_FP4_MX_GROUPED_MATMUL_ALLTOALLV, "Ascend950Fp4MxGroupedMatmulAllToAllV"},
        {ASCEND950_FP4_MX_ALLTOALLV_GROUPED_MATMUL, "Ascend950Fp4MxAllToAllVGroupedMatmul"},
    };
    return m;
}

inline int32_t CeilDev(int32_t num, int32_t div) { return div == 0 ? 0 : (num + div - 1) / div; }

#endif  // CATCCOS_HOST_INFO_H
