// Host-side operator classes of the fused operators: device buffers from raw .bin files, result
// files, workspace sizes, tiling checks — the same classes, names and file conventions as the
// reference's examples/<op>/<op>_host.h, on top of the CUDA runtime and the C-ABI.
#ifndef CATCCOS_HOST_OPERATORS_H
#define CATCCOS_HOST_OPERATORS_H

#include <vector>

#include "operator_registry.h"

namespace catccos_host {

// device buffer filled from `path` (or with `fill` repeated when path is empty / unreadable)
inline uint8_t *DeviceBufferFromFile(const std::string &path, size_t bytes, int fillByte = 0) {
    uint8_t *dev = nullptr;
    CUDA_CHECK(cudaMalloc(reinterpret_cast<void **>(&dev), bytes));
    std::vector<uint8_t> host(bytes, static_cast<uint8_t>(fillByte));
    if (!path.empty()) ReadFile(path, host.data(), bytes);
    CUDA_CHECK(cudaMemcpy(dev, host.data(), bytes, cudaMemcpyHostToDevice));
    return dev;
}
inline uint8_t *DeviceZeros(size_t bytes) {
    uint8_t *dev = nullptr;
    CUDA_CHECK(cudaMalloc(reinterpret_cast<void **>(&dev), bytes));
    CUDA_CHECK(cudaMemset(dev, 0, bytes));
    return dev;
}
inline void WriteDeviceBuffer(const std::string &path, const uint8_t *dev, size_t bytes, size_t offset = 0) {
    std::vector<uint8_t> host(bytes);
    CUDA_CHECK(cudaMemcpy(host.data(), dev, bytes, cudaMemcpyDeviceToHost));
    WriteFile(path, host.data(), bytes, offset);
}
inline std::string RankFile(const std::string &dir, const std::string &stem, uint32_t rank, const std::string &tail = "") {
    return dir.empty() ? std::string() : dir + "/" + stem + std::to_string(rank) + tail + ".bin";
}

// shapes the tcgen05 kernels take: n and k multiples of 8 (16-byte rows for TMA)
inline bool DenseShapeOk(const CocTilingParams &t) { return t.m > 0 && t.n > 0 && t.k > 0 && t.n % 8 == 0 && t.k % 8 == 0; }

}  // namespace catccos_host

// D = sum_r A_r * B_r on every rank (examples/matmul_allreduce/matmul_allreduce_host.h).
class MatmulAllReduceOperator : public CatccosOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t aSize = static_cast<size_t>(t.m) * t.k * 2, bSize = static_cast<size_t>(t.k) * t.n * 2;
        const size_t dSize = static_cast<size_t>(t.m) * t.n * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a"), aSize),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b"), bSize), DeviceZeros(dSize));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t, std::string dataFile) override {
        catccos_host::WriteDeviceBuffer(dataFile + "/output.bin", params.ptrC, static_cast<size_t>(t.m) * t.n * 2);
    }
    size_t GetWorkspaceSize(const CocTilingParams &) override { return 0; }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return MATMUL_ALLREDUCE; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return catccos_host::DenseShapeOk(t) && rankSize >= 1 && rankSize <= MAX_RANK_SIZE &&
               catccos_symmetric_bytes(MATMUL_ALLREDUCE, FP16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("MatmulAllReduce", MatmulAllReduceOperator);

// C[s*m:(s+1)*m] = A_s * B for all s (examples/allgather_matmul/allgather_matmul_host.h); m = rows per rank.
class AllGatherMatmulOperator : public CatccosOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t aSize = static_cast<size_t>(t.m) * t.k * 2, bSize = static_cast<size_t>(t.k) * t.n * 2;
        const size_t cSize = static_cast<size_t>(t.m) * t.rankSize * t.n * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a"), aSize),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b"), bSize), DeviceZeros(cSize));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        const size_t cSize = static_cast<size_t>(t.m) * t.rankSize * t.n * 2;
        // the reference writes one output.bin; per-rank weights give per-rank results, so each rank also
        // writes output_<rank>.bin
        catccos_host::WriteDeviceBuffer(dataFile + "/output_" + std::to_string(rankId) + ".bin", params.ptrC, cSize);
        if (rankId == 0) catccos_host::WriteDeviceBuffer(dataFile + "/output.bin", params.ptrC, cSize);
    }
    size_t GetWorkspaceSize(const CocTilingParams &) override { return 0; }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ALLGATHER_MATMUL; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return catccos_host::DenseShapeOk(t) && rankSize >= 1 && rankSize <= MAX_RANK_SIZE &&
               catccos_symmetric_bytes(ALLGATHER_MATMUL, BF16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("AllGatherMatmul", AllGatherMatmulOperator);
class Ascend950AllGatherMatmulOperator : public AllGatherMatmulOperator {
public:
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_ALLGATHER_MATMUL; }
};
REGISTER_OPERATOR("Ascend950AllGatherMatmul", Ascend950AllGatherMatmulOperator);
// The same product plus the gathered A [rankSize*m, k] in customPtrs[0], written to output_gather_a.bin
// (examples/allgather_matmul_with_gather_result/allgather_matmul_with_gather_result_host.h:17-84).
class AllGatherMatmulWithGatherResultOperator : public AllGatherMatmulOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t aSize = static_cast<size_t>(t.m) * t.k * 2, bSize = static_cast<size_t>(t.k) * t.n * 2;
        const size_t cSize = static_cast<size_t>(t.m) * t.rankSize * t.n * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a"), aSize),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b"), bSize), DeviceZeros(cSize),
                               DeviceZeros(aSize * t.rankSize));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        AllGatherMatmulOperator::WriteResultFile(params, t, rankId, dataFile);
        const size_t gSize = static_cast<size_t>(t.m) * t.rankSize * t.k * 2;
        catccos_host::WriteDeviceBuffer(dataFile + "/output_gather_a_" + std::to_string(rankId) + ".bin", params.customPtrs[0], gSize);
        if (rankId == 0) catccos_host::WriteDeviceBuffer(dataFile + "/output_gather_a.bin", params.customPtrs[0], gSize);
    }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ALLGATHER_MATMUL_WITH_GATHER_RESULT; }
};
REGISTER_OPERATOR("AllGatherMatmulWithGatherResult", AllGatherMatmulWithGatherResultOperator);
// Remote-read data flow (examples/allgather_matmul_remote_read/allgather_matmul_remote_read_host.h): same files.
class AllGatherMatmulRemoteReadOperator : public AllGatherMatmulOperator {
public:
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ALLGATHER_MATMUL_REMOTE_READ; }
};
REGISTER_OPERATOR("AllGatherMatmulRemoteRead", AllGatherMatmulRemoteReadOperator);
// AllToAll-Matmul (examples/ascend950_alltoall_matmul/ascend950_alltoall_matmul_host.h:17-109): A [m, k] per rank, block j
// of its rows goes to rank j; C [m, n] per rank, written to output_<rank>.bin.
class Ascend950AllToAllMatmulOperator : public CatccosOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t aSize = static_cast<size_t>(t.m) * t.k * 2, bSize = static_cast<size_t>(t.k) * t.n * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a"), aSize),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b"), bSize),
                               DeviceZeros(static_cast<size_t>(t.m) * t.n * 2));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        catccos_host::WriteDeviceBuffer(dataFile + "/output_" + std::to_string(rankId) + ".bin", params.ptrC,
                                        static_cast<size_t>(t.m) * t.n * 2);
    }
    size_t GetWorkspaceSize(const CocTilingParams &) override { return 0; }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_ALLTOALL_MATMUL; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return catccos_host::DenseShapeOk(t) && rankSize >= 1 && rankSize <= MAX_RANK_SIZE && t.m % rankSize == 0 &&
               catccos_symmetric_bytes(ASCEND950_ALLTOALL_MATMUL, BF16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("Ascend950AllToAllMatmul", Ascend950AllToAllMatmulOperator);
// Matmul-AllToAll (examples/ascend950_matmul_alltoall/ascend950_matmul_alltoall_host.h:17-100): C_i = A_i x B_i, then row
// block j of every C_i goes to rank j; same files and sizes as AllToAll-Matmul.
class Ascend950MatmulAllToAllOperator : public Ascend950AllToAllMatmulOperator {
public:
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_MATMUL_ALLTOALL; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return catccos_host::DenseShapeOk(t) && rankSize >= 1 && rankSize <= MAX_RANK_SIZE && t.m % rankSize == 0 &&
               catccos_symmetric_bytes(ASCEND950_MATMUL_ALLTOALL, BF16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("Ascend950MatmulAllToAll", Ascend950MatmulAllToAllOperator);

// D_r = rows r of sum_s A_s * B_s (examples/matmul_reduce_scatter/matmul_reduce_scatter_host.h); m = total rows.
class MatmulReduceScatterOperator : public CatccosOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t aSize = static_cast<size_t>(t.m) * t.k * 2, bSize = static_cast<size_t>(t.k) * t.n * 2;
        const size_t cSize = static_cast<size_t>(t.m) / t.rankSize * t.n * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a"), aSize),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b"), bSize), DeviceZeros(cSize));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        const size_t cSize = static_cast<size_t>(t.m) / t.rankSize * t.n * 2;
        catccos_host::WriteDeviceBuffer(dataFile + "/output.bin", params.ptrC, cSize, rankId * cSize);   // offset r*size
    }
    size_t GetWorkspaceSize(const CocTilingParams &) override { return 0; }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return MATMUL_REDUCE_SCATTER; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return catccos_host::DenseShapeOk(t) && rankSize >= 1 && rankSize <= MAX_RANK_SIZE && t.m % rankSize == 0 &&
               catccos_symmetric_bytes(MATMUL_REDUCE_SCATTER, BF16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("MatmulReduceScatter", MatmulReduceScatterOperator);
class Ascend950MatmulReduceScatterOperator : public MatmulReduceScatterOperator {
public:
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_MATMUL_REDUCE_SCATTER; }
};
REGISTER_OPERATOR("Ascend950MatmulReduceScatter", Ascend950MatmulReduceScatterOperator);

// MXFP8 AllGather-Matmul (examples/ascend950_fp8_mx_allgather_matmul/ascend950_fp8_mx_allgather_matmul_host.h):
// customPtrs = {aScale, bScale}.
class Ascend950Fp8MxAllGatherMatmulOperator : public CatccosOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t sizeA = static_cast<size_t>(t.m) * t.k, sizeB = static_cast<size_t>(t.k) * t.n;
        const size_t kb = (static_cast<size_t>(t.k) / 32 + 1) / 2 * 2;
        const size_t sizeC = static_cast<size_t>(t.m) * t.rankSize * t.n * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "input_a_", rankId), sizeA),
                               DeviceBufferFromFile(RankFile(dataFile, "input_b_", rankId), sizeB), DeviceZeros(sizeC),
                               DeviceBufferFromFile(RankFile(dataFile, "input_a_scale_", rankId), t.m * kb, 127),
                               DeviceBufferFromFile(RankFile(dataFile, "input_b_scale_", rankId), t.n * kb, 127));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        catccos_host::WriteDeviceBuffer(dataFile + "/output_" + std::to_string(rankId) + ".bin", params.ptrC,
                                        static_cast<size_t>(t.m) * t.rankSize * t.n * 2);
    }
    size_t GetWorkspaceSize(const CocTilingParams &t) override {
        return catccos_workspace_bytes(ASCEND950_FP8_MX_ALLGATHER_MATMUL, FP16, &t);
    }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_FP8_MX_ALLGATHER_MATMUL; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return t.m > 0 && t.k % 32 == 0 && t.n % 16 == 0 && rankSize <= MAX_RANK_SIZE &&
               catccos_symmetric_bytes(ASCEND950_FP8_MX_ALLGATHER_MATMUL, FP16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("Ascend950Fp8MxAllGatherMatmul", Ascend950Fp8MxAllGatherMatmulOperator);

// MXFP4 AllGather-Matmul (examples/ascend950_fp4_mx_allgather_matmul/ascend950_fp4_mx_allgather_matmul_host.h:17-140):
// e2m1 codes packed two per byte, A [m, k/2], B^T [n, k/2] (run with transB = 1), E8M0 scales per 32 along k.
class Ascend950Fp4MxAllGatherMatmulOperator : public CatccosOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t sizeA = static_cast<size_t>(t.m) * t.k / 2, sizeB = static_cast<size_t>(t.k) / 2 * t.n;
        const size_t kb = (static_cast<size_t>(t.k) / 32 + 1) / 2 * 2;
        const size_t sizeC = static_cast<size_t>(t.m) * t.rankSize * t.n * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "input_a_", rankId), sizeA),
                               DeviceBufferFromFile(RankFile(dataFile, "input_b_", rankId), sizeB), DeviceZeros(sizeC),
                               DeviceBufferFromFile(RankFile(dataFile, "input_a_scale_", rankId), t.m * kb, 127),
                               DeviceBufferFromFile(RankFile(dataFile, "input_b_scale_", rankId), t.n * kb, 127));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        catccos_host::WriteDeviceBuffer(dataFile + "/output_" + std::to_string(rankId) + ".bin", params.ptrC,
                                        static_cast<size_t>(t.m) * t.rankSize * t.n * 2);
    }
    size_t GetWorkspaceSize(const CocTilingParams &t) override {
        return catccos_workspace_bytes(ASCEND950_FP4_MX_ALLGATHER_MATMUL, FP16, &t);
    }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_FP4_MX_ALLGATHER_MATMUL; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return t.m > 0 && t.k % 64 == 0 && t.n % 16 == 0 && rankSize <= MAX_RANK_SIZE &&
               catccos_symmetric_bytes(ASCEND950_FP4_MX_ALLGATHER_MATMUL, FP16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("Ascend950Fp4MxAllGatherMatmul", Ascend950Fp4MxAllGatherMatmulOperator);

// MXFP4 Matmul-ReduceScatter (examples/ascend950_fp4_mx_matmul_reduce_scatter/ascend950_fp4_mx_matmul_reduce_scatter_host.h:17-110):
// rank_<i>_{a,b}[_scale].bin, rank r's rows at offset r*size of output.bin.  B as B^T [n, k/2] (run with transB = 1).
class Ascend950Fp4MxMatmulReduceScatterOperator : public CatccosOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t sizeA = static_cast<size_t>(t.m) * t.k / 2, sizeB = static_cast<size_t>(t.k) / 2 * t.n;
        const size_t kb = (static_cast<size_t>(t.k) + 63) / 64 * 2;
        const size_t sizeC = static_cast<size_t>(t.m) * t.n / t.rankSize * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a"), sizeA),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b"), sizeB), DeviceZeros(sizeC),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a_scale"), t.m * kb, 127),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b_scale"), t.n * kb, 127));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        const size_t cSize = static_cast<size_t>(t.m) * t.n / t.rankSize * 2;
        catccos_host::WriteDeviceBuffer(dataFile + "/output.bin", params.ptrC, cSize, rankId * cSize);
    }
    size_t GetWorkspaceSize(const CocTilingParams &t) override {
        return catccos_workspace_bytes(ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER, BF16, &t);
    }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return t.m > 0 && t.k % 64 == 0 && t.n % 16 == 0 && rankSize >= 1 && rankSize <= MAX_RANK_SIZE &&
               t.m % rankSize == 0 && (t.m / rankSize) % 128 == 0 &&
               catccos_symmetric_bytes(ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER, BF16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("Ascend950Fp4MxMatmulReduceScatter", Ascend950Fp4MxMatmulReduceScatterOperator);

// MXFP8 Matmul-ReduceScatter (examples/ascend950_mxfp8_matmul_reduce_scatter/ascend950_mxfp8_matmul_reduce_scatter_host.h):
// float8_e5m2 operands, customPtrs = {aScale, bScale}, rank r's rows written at offset r*size of output.bin.
class Ascend950MxFp8MatmulReduceScatterOperator : public CatccosOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t sizeA = static_cast<size_t>(t.m) * t.k, sizeB = static_cast<size_t>(t.k) * t.n;
        const size_t kb = (static_cast<size_t>(t.k) + 63) / 64 * 2;
        const size_t sizeC = static_cast<size_t>(t.m) * t.n / t.rankSize * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a"), sizeA, 60),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b"), sizeB, 60), DeviceZeros(sizeC),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a_scale"), t.m * kb, 121),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b_scale"), t.n * kb, 121));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        const size_t cSize = static_cast<size_t>(t.m) * t.n / t.rankSize * 2;
        catccos_host::WriteDeviceBuffer(dataFile + "/output.bin", params.ptrC, cSize, rankId * cSize);
    }
    size_t GetWorkspaceSize(const CocTilingParams &t) override {
        return catccos_workspace_bytes(ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER, BF16, &t);
    }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return t.m > 0 && t.k % 32 == 0 && t.n % 16 == 0 && rankSize >= 1 && rankSize <= MAX_RANK_SIZE &&
               t.m % rankSize == 0 && (t.m / rankSize) % 128 == 0 &&
               catccos_symmetric_bytes(ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER, BF16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("Ascend950MxFp8MatmulReduceScatter", Ascend950MxFp8MatmulReduceScatterOperator);
// MXFP8 Matmul-AllToAll (examples/ascend950_mxfp8_matmul_alltoall/ascend950_mxfp8_matmul_alltoall_host.h:17-120, row-block
// form): e4m3 operands and scales in the files of the operator above, C [m, n] written to output_<rank>.bin.
class Ascend950MxFp8MatmulAllToAllOperator : public Ascend950MxFp8MatmulReduceScatterOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t sizeA = static_cast<size_t>(t.m) * t.k, sizeB = static_cast<size_t>(t.k) * t.n;
        const size_t kb = (static_cast<size_t>(t.k) + 63) / 64 * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a"), sizeA, 56),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b"), sizeB, 56),
                               DeviceZeros(static_cast<size_t>(t.m) * t.n * 2),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_a_scale"), t.m * kb, 121),
                               DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_b_scale"), t.n * kb, 121));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        catccos_host::WriteDeviceBuffer(dataFile + "/output_" + std::to_string(rankId) + ".bin", params.ptrC,
                                        static_cast<size_t>(t.m) * t.n * 2);
    }
    size_t GetWorkspaceSize(const CocTilingParams &t) override {
        return catccos_workspace_bytes(ASCEND950_MXFP8_MATMUL_ALLTOALL, BF16, &t);
    }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_MXFP8_MATMUL_ALLTOALL; }
};
REGISTER_OPERATOR("Ascend950MxFp8MatmulAllToAll", Ascend950MxFp8MatmulAllToAllOperator);

// MoE dispatch -> FFN -> combine (examples/ascend950_dispatch_ffn_combine/ascend950_dispatch_ffn_combine_host.h):
// customPtrs = {b2, expertIdx, probs, bScale, b2Scale}.
class Ascend950DispatchFFNCombineOperator : public CatccosOperator {
public:
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t el = t.expertNum / (t.epSize ? t.epSize : t.rankSize);
        const size_t aSize = static_cast<size_t>(t.m) * t.k * 2, cSize = aSize;
        const size_t bSize = el * t.n * t.k, b2Size = el * t.k * (t.n / 2);
        const size_t bScaleSize = el * t.n * (t.k / 32), b2ScaleSize = el * t.k * (t.n / 2 / 32);
        const size_t idxSize = static_cast<size_t>(t.m) * t.topK * 4;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "in_routing_matrix_a_", rankId), aSize),
                               DeviceBufferFromFile(RankFile(dataFile, "in_gmm_matrix_b_", rankId), bSize), DeviceZeros(cSize),
                               DeviceBufferFromFile(RankFile(dataFile, "in_gmm_matrix_b2_", rankId), b2Size),
                               DeviceBufferFromFile(RankFile(dataFile, "in_routing_expert_idx_", rankId), idxSize),
                               DeviceBufferFromFile(RankFile(dataFile, "in_gather_gate_weight_", rankId), idxSize),
                               DeviceBufferFromFile(RankFile(dataFile, "in_gmm_matrix_b_scale_", rankId), bScaleSize, 127),
                               DeviceBufferFromFile(RankFile(dataFile, "in_gmm_matrix_b2_scale_", rankId), b2ScaleSize, 127));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        catccos_host::WriteDeviceBuffer(dataFile + "/output_" + std::to_string(rankId) + ".bin", params.ptrC,
                                        static_cast<size_t>(t.m) * t.k * 2);
    }
    size_t GetWorkspaceSize(const CocTilingParams &t) override {
        return catccos_workspace_bytes(ASCEND950_DISPATCH_FFN_COMBINE, BF16, &t);
    }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_DISPATCH_FFN_COMBINE; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        if (t.k % 256 != 0 || t.n % 512 != 0) {
            std::fprintf(stderr, "MXFP8 FFN requires K %% 256 == 0 and N %% 512 == 0\n");
            return false;
        }
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return t.expertNum > 0 && t.expertNum % rankSize == 0 && t.topK >= 1 && t.topK <= 16 &&
               catccos_symmetric_bytes(ASCEND950_DISPATCH_FFN_COMBINE, BF16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("Ascend950DispatchFFNCombine", Ascend950DispatchFFNCombineOperator);

// MX quantisation + all-gather (examples/ascend950_mx_quant_allgather/mx_quant_allgather_host.h:48-74): every rank
// quantises its bf16 [m, n] input to e4m3 + one E8M0 scale per 32 along n and ends with all ranks' codes
// (ptrC, [rankSize*m, n]) and scales (ptrB, [rankSize*m, even(n/32)]).  Files: rank_<r>_input.bin in,
// rank_<r>_output.bin and rank_<r>_mxscale.bin out.
class MxQuantAllGatherOperator : public CatccosOperator {
public:
    static constexpr uint32_t MX_BLOCK_SIZE = 32;
    static size_t ScalesPerRow(uint32_t n) { return (static_cast<size_t>(n) / MX_BLOCK_SIZE + 1) / 2 * 2; }
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t inputSize = static_cast<size_t>(t.m) * t.n * 2;
        const size_t outputSize = static_cast<size_t>(t.m) * t.n * t.rankSize;
        const size_t scaleSize = static_cast<size_t>(t.m) * ScalesPerRow(t.n) * t.rankSize;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, "rank_", rankId, "_input"), inputSize),
                               DeviceZeros(scaleSize), DeviceZeros(outputSize));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        catccos_host::WriteDeviceBuffer(dataFile + "/rank_" + std::to_string(rankId) + "_output.bin", params.ptrC,
                                        static_cast<size_t>(t.m) * t.n * t.rankSize);
        catccos_host::WriteDeviceBuffer(dataFile + "/rank_" + std::to_string(rankId) + "_mxscale.bin", params.ptrB,
                                        static_cast<size_t>(t.m) * ScalesPerRow(t.n) * t.rankSize);
    }
    size_t GetWorkspaceSize(const CocTilingParams &) override { return 0; }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return MX_QUANT_ALLGATHER; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        if (t.m == 0 || t.n == 0 || t.n % MX_BLOCK_SIZE != 0) return false;
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return rankSize >= 1 && rankSize <= MAX_RANK_SIZE &&
               catccos_symmetric_bytes(MX_QUANT_ALLGATHER, FP8E4M3FN, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("MxQuantAllGather", MxQuantAllGatherOperator);

// Standalone MXFP8 AllToAllV-GroupedMatmul (examples/ascend950_fp8_mx_alltoallv_grouped_matmul/..._host.h:14-156) and
// GroupedMatmul-AllToAllV (examples/ascend950_fp8_mx_grouped_matmul_alltoallv/..._host.h): customPtrs = {aScale,
// bScale, localTokensPerExpert, globalTokensPerLocalExpert}; output_<rank>.bin holds [rankSize*m, n] 16-bit rows.
class Ascend950Fp8MxAllToAllVGroupedMatmulOperator : public CatccosOperator {
public:
    virtual const char *AName() const { return "input_a_"; }
    virtual const char *BName() const { return "input_b_"; }
    virtual const char *AScaleName() const { return "input_a_scale_"; }
    virtual const char *BScaleName() const { return "input_b_scale_"; }
    virtual size_t CodesPerByte() const { return 1; }      // 2 for the MXFP4 operators
    void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        using namespace catccos_host;
        const size_t el = t.expertNum / (t.epSize ? t.epSize : t.rankSize);
        const size_t kb = static_cast<size_t>(t.k) / 32;
        const size_t sizeA = static_cast<size_t>(t.m) * t.k / CodesPerByte(), sizeB = el * t.k * t.n / CodesPerByte();
        const size_t sizeC = static_cast<size_t>(t.m) * t.rankSize * t.n * 2;
        params.SetKernelParams(DeviceBufferFromFile(RankFile(dataFile, AName(), rankId), sizeA),
                               DeviceBufferFromFile(RankFile(dataFile, BName(), rankId), sizeB), DeviceZeros(sizeC),
                               DeviceBufferFromFile(RankFile(dataFile, AScaleName(), rankId), t.m * kb, 127),
                               DeviceBufferFromFile(RankFile(dataFile, BScaleName(), rankId), el * kb * t.n, 127),
                               DeviceBufferFromFile(RankFile(dataFile, "local_tokens_per_expert_", rankId), t.expertNum * 4),
                               DeviceBufferFromFile(RankFile(dataFile, "global_tokens_per_local_expert_", rankId),
                                                    static_cast<size_t>(t.rankSize) * el * 4));
    }
    void WriteResultFile(const KernelParams &params, const CocTilingParams &t, uint32_t rankId, std::string dataFile) override {
        catccos_host::WriteDeviceBuffer(dataFile + "/output_" + std::to_string(rankId) + ".bin", params.ptrC,
                                        static_cast<size_t>(t.m) * t.rankSize * t.n * 2);
    }
    size_t GetWorkspaceSize(const CocTilingParams &t) override { return catccos_workspace_bytes(GetActualKernelType(t), FP16, &t); }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_FP8_MX_ALLTOALLV_GROUPED_MATMUL; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        CocTilingParams c = t;
        c.rankSize = rankSize;
        return t.m > 0 && t.k % 64 == 0 && t.n % 16 == 0 && t.expertNum > 0 && t.expertNum % rankSize == 0 &&
               (t.epSize == 0 || t.epSize == rankSize) && rankSize <= MAX_RANK_SIZE &&
               catccos_symmetric_bytes(GetActualKernelType(t), FP16, &c) <= SHMEM_BUFF_BYTES;
    }
};
REGISTER_OPERATOR("Ascend950Fp8MxAllToAllVGroupedMatmul", Ascend950Fp8MxAllToAllVGroupedMatmulOperator);
class Ascend950Fp8MxGroupedMatmulAllToAllVOperator : public Ascend950Fp8MxAllToAllVGroupedMatmulOperator {
public:
    const char *AName() const override { return "a_gm_"; }
    const char *BName() const override { return "b_gm_"; }
    const char *AScaleName() const override { return "a_scale_"; }
    const char *BScaleName() const override { return "b_scale_"; }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_FP8_MX_GROUPED_MATMUL_ALLTOALLV; }
};
REGISTER_OPERATOR("Ascend950Fp8MxGroupedMatmulAllToAllV", Ascend950Fp8MxGroupedMatmulAllToAllVOperator);
// The MXFP4 forms (examples/ascend950_fp4_mx_alltoallv_grouped_matmul, examples/ascend950_fp4_mx_grouped_matmul_alltoallv):
// the same files with two e2m1 codes per byte; weights K-major (generated with transB = 1), k % 256 == 0.
class Ascend950Fp4MxAllToAllVGroupedMatmulOperator : public Ascend950Fp8MxAllToAllVGroupedMatmulOperator {
public:
    size_t CodesPerByte() const override { return 2; }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_FP4_MX_ALLTOALLV_GROUPED_MATMUL; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        return t.k % 256 == 0 && Ascend950Fp8MxAllToAllVGroupedMatmulOperator::CheckCocTilingParams(rankSize, t);
    }
};
REGISTER_OPERATOR("Ascend950Fp4MxAllToAllVGroupedMatmul", Ascend950Fp4MxAllToAllVGroupedMatmulOperator);
class Ascend950Fp4MxGroupedMatmulAllToAllVOperator : public Ascend950Fp8MxGroupedMatmulAllToAllVOperator {
public:
    size_t CodesPerByte() const override { return 2; }
    CocCommType GetActualKernelType(const CocTilingParams &) override { return ASCEND950_FP4_MX_GROUPED_MATMUL_ALLTOALLV; }
    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &t) override {
        return t.k % 256 == 0 && Ascend950Fp8MxGroupedMatmulAllToAllVOperator::CheckCocTilingParams(rankSize, t);
    }
};
REGISTER_OPERATOR("Ascend950Fp4MxGroupedMatmulAllToAllV", Ascend950Fp4MxGroupedMatmulAllToAllVOperator);

#endif  // CATCCOS_HOST_OPERATORS_H
