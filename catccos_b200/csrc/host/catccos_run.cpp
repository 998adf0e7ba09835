// One rank of one fused operator, driven the way the reference's per-example main.cpp and its
// dynamic-tiling launcher drive it (examples/matmul_allreduce/main.cpp:27-178,
// tests/dynamic_tiling/main.cpp:200-368): symmetric-heap init, operator from the registry,
// AllocateDeviceSpace from .bin files, launcher from the (commType, dataType) map, warm-up and
// timed launches, WriteResultFile.
//
//   catccos_run <kernel> <dtype> <rank_size> <rank_id> <ip_port> <m> <n> <k> <data_dir>
//               [transA transB [topK expertNum [device_id [warmup timed]]]]
//   kernel: mmar | agmm | a5agmm | mmrs | a5mmrs | a5fp8mxagmm | a5mxfp8mmrs | a5moe | mxqtag | a5fp8mxatavgmm | a5fp8gmmata | agmmwg | agmmrr | a5fp4mxagmm | a5atamm | a5mmata | a5mxfp8mmata | a5fp4mmrs | a5fp4mxatavgmm | a5fp4gmmata
//   dtype: 1 (fp16) | 27 (bf16) | 36 (float8_e4m3fn, mxqtag)
//   catccos_run --list        prints the registered operator names
//   catccos_run --check <kernel> <rank_size> <m> <n> <k> [topK expertNum]
//                             CheckCocTilingParams + symmetric / workspace bytes, no device needed
//   catccos_run --tilings <kernel> <rank_size> <m> <n> <k> <csv>
//                             the operator's tiling candidates with the model's prediction, as a CSV
//   catccos_run --estimate <kernel> <rank_size> <m> <n> <k> [m0 blockNum]
//                             the B200 cost model's tiling choice and predicted time, no device needed
#include <cuda_runtime.h>

#include <cstdlib>
#include <iostream>
#include <string>

#include "catccos_host/cost_model.h"
#include "catccos_host/launch_map.h"
#include "catccos_host/operators.h"
#include "catccos_host/tiling.h"

int main(int argc, char **argv) {
    if (argc >= 2 && std::string(argv[1]) == "--list") {
        for (const auto &n : OperatorRegistry::Instance().Names()) std::cout << n << "\n";
        return 0;
    }
    if (argc >= 8 && std::string(argv[1]) == "--tilings") {
        // catccos_run --tilings <kernel> <rank_size> <m> <n> <k> <csv>: writes the tiling candidates of the operator
        // (those its CheckCocTilingParams accepts) with the cost model's prediction, one CSV row each
        const CocCommType ct = GetCommType(argv[2]);
        if (ct == UNKNOWN) {
            std::cerr << "unknown kernel " << argv[2] << "\n";
            return 1;
        }
        CocTilingParams t{};
        t.m = static_cast<uint32_t>(std::atoi(argv[4]));
        t.n = static_cast<uint32_t>(std::atoi(argv[5]));
        t.k = static_cast<uint32_t>(std::atoi(argv[6]));
        t.topK = 1;
        t.epSize = static_cast<uint32_t>(std::atoi(argv[3]));
        std::vector<TilingCandidate> cands;
        const std::string opName = CommTypeOpNameMap().at(ct);
        GetTilings(cands, t, opName, std::atoi(argv[3]));
        if (!CreateTilingFile(argv[7]) || !WriteTilingInfos(opName, cands, argv[7])) return 1;
        std::cout << cands.size() << "\n";
        return 0;
    }
    if (argc >= 7 && std::string(argv[1]) == "--estimate") {
        // catccos_run --estimate <kernel> <rank_size> <m> <n> <k> [m0 blockNum]: the cost model's choice (or the
        // cost of the given candidate): "m0 blockNum cost_us compute_us comm_us"
        const CocCommType ct = GetCommType(argv[2]);
        const uint32_t rs = static_cast<uint32_t>(std::atoi(argv[3]));
        const COCMatMulInfo info{std::atoll(argv[4]), std::atoll(argv[6]), std::atoll(argv[5])};
        CostModelResult r;
        if (argc >= 9) {
            catccos_cost::Family family;
            bool mx;
            if (ct == UNKNOWN || !catccos_cost::FamilyOf(ct, family, mx)) {
                std::cout << "unsupported\n";
                return 2;
            }
            CostModelTiling t;
            t.m0 = static_cast<uint32_t>(std::atoi(argv[7]));
            t.n0 = 256;
            t.k0 = mx ? 128 : 64;
            t.blockNum = static_cast<uint32_t>(std::atoi(argv[8]));
            r = catccos_cost::Evaluate(info, family, mx, rs, t, CostModelHardwareConfig{});
        } else {
            r = ct == UNKNOWN ? CostModelResult{} : SelectCostModelTiling(info, ct, rs);
        }
        if (!r.IsSuccess()) {
            std::cout << (r.status == CostModelStatus::UNSUPPORTED ? "unsupported" : "invalid") << "\n";
            return 2;
        }
        std::printf("%u %u %.2f %.2f %.2f\n", r.tiling.m0, r.tiling.blockNum, r.cost, r.computeUs, r.commUs);
        return 0;
    }
    if (argc >= 7 && std::string(argv[1]) == "--check") {
        // catccos_run --check <kernel> <rank_size> <m> <n> <k> [topK expertNum]: the operator's tiling check and
        // buffer sizes, without touching a device
        const CocCommType ct = GetCommType(argv[2]);
        if (ct == UNKNOWN) {
            std::cerr << "unknown kernel " << argv[2] << "\n";
            return 1;
        }
        auto chk = OperatorRegistry::Instance().CreateOperator(CommTypeOpNameMap().at(ct));
        if (!chk) return 1;
        CocTilingParams t{};
        const int rs = std::atoi(argv[3]);
        t.m = static_cast<uint32_t>(std::atoi(argv[4]));
        t.n = static_cast<uint32_t>(std::atoi(argv[5]));
        t.k = static_cast<uint32_t>(std::atoi(argv[6]));
        t.topK = argc > 7 ? std::atoi(argv[7]) : 1;
        t.expertNum = argc > 8 ? std::atoi(argv[8]) : 0;
        t.m0 = M0;
        t.n0 = N0;
        t.k0 = K0;
        t.rankSize = rs;
        t.epSize = rs;
        if (rs < 1 || !chk->CheckCocTilingParams(static_cast<uint32_t>(rs), t)) {
            std::cout << "rejected\n";
            return 2;
        }
        const CocCommType actual = chk->GetActualKernelType(t);
        std::cout << "ok " << catccos_symmetric_bytes(actual, BF16, &t) << " " << chk->GetWorkspaceSize(t) << "\n";
        return 0;
    }
    if (argc < 10) {
        std::cerr << "usage: catccos_run <kernel> <dtype> <rank_size> <rank_id> <ip_port> <m> <n> <k> <data_dir> "
                     "[transA transB [topK expertNum [device_id [warmup timed]]]]\n";
        return 1;
    }
    const std::string kernel = argv[1];
    const CocDataType dtype = static_cast<CocDataType>(std::atoi(argv[2]));
    const int rankSize = std::atoi(argv[3]), rankId = std::atoi(argv[4]);
    const std::string ipPort = argv[5];
    CocTilingParams tiling{};
    tiling.m = static_cast<uint32_t>(std::atoi(argv[6]));
    tiling.n = static_cast<uint32_t>(std::atoi(argv[7]));
    tiling.k = static_cast<uint32_t>(std::atoi(argv[8]));
    const std::string dataDir = argv[9];
    tiling.transA = argc > 10 ? std::atoi(argv[10]) : 0;
    tiling.transB = argc > 11 ? std::atoi(argv[11]) : 0;
    tiling.topK = argc > 12 ? std::atoi(argv[12]) : 1;
    tiling.expertNum = argc > 13 ? std::atoi(argv[13]) : 0;
    const int deviceId = argc > 14 ? std::atoi(argv[14]) : rankId;
    const int warmUp = argc > 15 ? std::atoi(argv[15]) : 0;
    const int timed = argc > 16 ? std::atoi(argv[16]) : 1;
    tiling.m0 = M0;
    tiling.n0 = N0;
    tiling.k0 = K0;
    tiling.rankSize = rankSize;
    tiling.epSize = rankSize;

    const CocCommType commType = GetCommType(kernel);
    if (commType == UNKNOWN) {
        std::cerr << "unknown kernel " << kernel << "\n";
        return 1;
    }
    auto op = OperatorRegistry::Instance().CreateOperator(CommTypeOpNameMap().at(commType));
    if (!op) {
        std::cout << "Operator " << CommTypeOpNameMap().at(commType) << " not found!" << std::endl;
        return -1;
    }
    std::cout << "[TEST] input rank_size: " << rankSize << " rank_id: " << rankId << " input_ip: " << ipPort << "\n";
    CUDA_CHECK(cudaSetDevice(deviceId));
    cudaStream_t stream = nullptr;
    CUDA_CHECK(cudaStreamCreate(&stream));
    if (catccos_shmem_init(rankId, rankSize, SHMEM_MALLOC_MAX_SIZE, ipPort.c_str()) != CATCCOS_OK) {
        std::cerr << "[ERROR] shmem init failed: " << catccos_last_error() << "\n";
        return 1;
    }
    if (!op->CheckCocTilingParams(rankSize, tiling)) {
        std::printf("M: %u, K: %u, N: %u coc params check failed!\n", tiling.m, tiling.k, tiling.n);
        catccos_shmem_finalize();
        return 1;
    }
    const CocCommType actual = op->GetActualKernelType(tiling);
    KernelParams params;
    op->AllocateDeviceSpace(params, tiling, rankId, dataDir);
    const size_t wsBytes = op->GetWorkspaceSize(tiling);
    uint8_t *workspace = nullptr;
    if (wsBytes > 0) CUDA_CHECK(cudaMalloc(reinterpret_cast<void **>(&workspace), wsBytes));
    uint8_t *symmetric = static_cast<uint8_t *>(catccos_shmem_malloc(SHMEM_BUFF_BYTES));
    const KernelFuncPtr launch = KernelDispatcher::GetKernelFunc(actual, dtype);
    int rc = 1;
    if (!symmetric) {
        std::cerr << "[ERROR] " << catccos_last_error() << "\n";
    } else if (!launch) {
        std::cerr << "[ERROR] no kernel registered for (" << actual << ", " << dtype << ")\n";
    } else {
        rc = 0;
        cudaEvent_t e0, e1;
        CUDA_CHECK(cudaEventCreate(&e0));
        CUDA_CHECK(cudaEventCreate(&e1));
        for (int i = 0; i < warmUp + timed && rc == 0; ++i) {
            if (i == warmUp) CUDA_CHECK(cudaEventRecord(e0, stream));
            rc = launch(stream, 0, 0, &params, workspace, symmetric, &tiling, tiling.transA, tiling.transB);
        }
        CUDA_CHECK(cudaEventRecord(e1, stream));
        if (rc != 0) std::cerr << "[ERROR] launch failed: " << catccos_last_error() << "\n";
        int32_t words[8];
        const int st = catccos_last_status(words);          // synchronises the device
        if (st != CATCCOS_OK) {
            std::cerr << "[ERROR] " << catccos_last_error() << "\n";
            rc = st;
        } else if (rc == 0) {
            float ms = 0;
            CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
            std::printf("[TEST] %s rank %d: %.3f us per launch (%d timed)\n", kernel.c_str(), rankId, ms * 1e3f / timed, timed);
            op->WriteResultFile(params, tiling, rankId, dataDir);
        }
    }
    catccos_shmem_barrier_all();
    FreeDeviceSpace(params);
    if (workspace) CUDA_CHECK(cudaFree(workspace));
    if (symmetric) catccos_shmem_free(symmetric);
    catccos_shmem_finalize();
    CUDA_CHECK(cudaStreamDestroy(stream));
    return rc;
}
