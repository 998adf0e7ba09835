// (CocCommType, CocDataType) -> launcher, the role of tests/dynamic_tiling/include/launch_map.h:15-59.
#ifndef CATCCOS_HOST_LAUNCH_MAP_H
#define CATCCOS_HOST_LAUNCH_MAP_H

#include <unordered_map>

#include "info.h"

// The reference's KernelFuncPtr with references replaced by pointers and an int status.
using KernelFuncPtr = int (*)(void *stream, uint32_t blockNum, uint64_t fftsAddr, CatccosKernelParams *, uint8_t *workspace,
                              uint8_t *symmetric, CocTilingParams *, uint32_t transA, uint32_t transB);

class KernelDispatcher {
public:
    static KernelFuncPtr GetKernelFunc(CocCommType commType, CocDataType dataType) {
        const auto &m = Map();
        const auto it = m.find(Hash(commType, dataType));
        return it == m.end() ? nullptr : it->second;
    }

private:
    static int Hash(CocCommType c, CocDataType d) { return (static_cast<int>(c) << 8) | static_cast<int>(d); }
    static const std::unordered_map<int, KernelFuncPtr> &Map() {
        static const std::unordered_map<int, KernelFuncPtr> m = {
            {Hash(MATMUL_ALLREDUCE, FP16), &LaunchMatmulAllReduceFP16},
            {Hash(MATMUL_ALLREDUCE, BF16), &LaunchMatmulAllReduceBF16},
            {Hash(ALLGATHER_MATMUL, FP16), &LaunchAllGatherMatmulFP16},
            {Hash(ALLGATHER_MATMUL, BF16), &LaunchAllGatherMatmulBF16},
            {Hash(ALLGATHER_MATMUL_WITH_GATHER_RESULT, FP16), &LaunchAllGatherMatmulWithGatherResultFP16},
            {Hash(ALLGATHER_MATMUL_WITH_GATHER_RESULT, BF16), &LaunchAllGatherMatmulWithGatherResultBF16},
            {Hash(ALLGATHER_MATMUL_REMOTE_READ, FP16), &LaunchAllGatherMatmulRemoteReadFP16},
            {Hash(ALLGATHER_MATMUL_REMOTE_READ, BF16), &LaunchAllGatherMatmulRemoteReadBF16},
            {Hash(ASCEND950_MATMUL_ALLTOALL, FP16), &LaunchAscend950MatmulAllToAllFP16},
            {Hash(ASCEND950_MATMUL_ALLTOALL, BF16), &LaunchAscend950MatmulAllToAllBF16},
            {Hash(ASCEND950_ALLTOALL_MATMUL, FP16), &LaunchAscend950AllToAllMatmulFP16},
            {Hash(ASCEND950_ALLTOALL_MATMUL, BF16), &LaunchAscend950AllToAllMatmulBF16},
            {Hash(MATMUL_REDUCE_SCATTER, FP16), &LaunchMatmulReduceScatterFP16},
            {Hash(MATMUL_REDUCE_SCATTER, BF16), &LaunchMatmulReduceScatterBF16},
            {Hash(ASCEND950_ALLGATHER_MATMUL, FP16), &LaunchAscend950AllGatherMatmulFP16},
            {Hash(ASCEND950_ALLGATHER_MATMUL, BF16), &LaunchAscend950AllGatherMatmulBF16},
            {Hash(ASCEND950_MATMUL_REDUCE_SCATTER, FP16), &LaunchAscend950MatmulReduceScatterFP16},
            {Hash(ASCEND950_MATMUL_REDUCE_SCATTER, BF16), &LaunchAscend950MatmulReduceScatterBF16},
            {Hash(ASCEND950_FP8_MX_ALLGATHER_MATMUL, FP16), &LaunchAscend950Fp8MxAllGatherMatmulFP16},
            {Hash(ASCEND950_FP8_MX_ALLGATHER_MATMUL, BF16), &LaunchAscend950Fp8MxAllGatherMatmulBF16},
            {Hash(ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER, FP16), &LaunchAscend950Fp4MxMatmulReduceScatterFP16},
            {Hash(ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER, BF16), &LaunchAscend950Fp4MxMatmulReduceScatterBF16},
            {Hash(ASCEND950_FP4_MX_ALLGATHER_MATMUL, FP16), &LaunchAscend950Fp4MxAllGatherMatmulFP16},
            {Hash(ASCEND950_FP4_MX_ALLGATHER_MATMUL, BF16), &LaunchAscend950Fp4MxAllGatherMatmulBF16},
            {Hash(ASCEND950_MXFP8_MATMUL_ALLTOALL, FP16), &LaunchAscend950MxFp8MatmulAllToAllFP16},
            {Hash(ASCEND950_MXFP8_MATMUL_ALLTOALL, BF16), &LaunchAscend950MxFp8MatmulAllToAllBF16},
            {Hash(ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER, FP16), &LaunchAscend950MxFp8MatmulReduceScatterFP16},
            {Hash(ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER, BF16), &LaunchAscend950MxFp8MatmulReduceScatterBF16},
            {Hash(ASCEND950_DISPATCH_FFN_COMBINE, BF16), &LaunchAscend950DispatchFFNCombineBF16},
            {Hash(MX_QUANT_ALLGATHER, FP8E4M3FN), &LaunchAscend950BF16QuantAllGatherFP8E4M3FN},
            {Hash(ASCEND950_FP4_MX_ALLTOALLV_GROUPED_MATMUL, FP16), &LaunchAscend950Fp4MxAllToAllVGroupedMatmulFP16},
            {Hash(ASCEND950_FP4_MX_ALLTOALLV_GROUPED_MATMUL, BF16), &LaunchAscend950Fp4MxAllToAllVGroupedMatmulBF16},
            {Hash(ASCEND950_FP4_MX_GROUPED_MATMUL_ALLTOALLV, FP16), &LaunchAscend950Fp4MxGroupedMatmulAllToAllVFP16},
            {Hash(ASCEND950_FP4_MX_GROUPED_MATMUL_ALLTOALLV, BF16), &LaunchAscend950Fp4MxGroupedMatmulAllToAllVBF16},
            {Hash(ASCEND950_FP8_MX_ALLTOALLV_GROUPED_MATMUL, FP16), &LaunchAscend950Fp8MxAllToAllVGroupedMatmulFP16},
            {Hash(ASCEND950_FP8_MX_ALLTOALLV_GROUPED_MATMUL, BF16), &LaunchAscend950Fp8MxAllToAllVGroupedMatmulBF16},
            {Hash(ASCEND950_FP8_MX_GROUPED_MATMUL_ALLTOALLV, FP16), &LaunchAscend950Fp8MxGroupedMatmulAllToAllVFP16},
            {Hash(ASCEND950_FP8_MX_GROUPED_MATMUL_ALLTOALLV, BF16), &LaunchAscend950Fp8MxGroupedMatmulAllToAllVBF16},
        };
        return m;
    }
};

#endif  // CATCCOS_HOST_LAUNCH_MAP_H
