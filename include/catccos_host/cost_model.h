// Analytic cost model of the fused operators on B200 and the tiling choice it drives.
//
// Counterpart of the reference's tests/dynamic_tiling (search space include/tiling.h:21-26, model
// include/cost_model.h:19-140 and tiling/*_cost_model.cpp, entry points SelectAllGatherTiling /
// SelectReduceScatterTiling / SelectAllReduceTiling / SelectCostModelTiling / ApplyCostModel).
// The reference searches commInterval x commTileM x m0 x (commNpuSplit, commDataSplit): the size
// of its communication windows and the split of vector cores between ranks and data.  The B200
// kernels have no windows and no core split (every GEMM CTA moves its own share of the traffic),
// so the search space here is what those kernels can actually vary:
//   * the tile: one CTA per 128 x 256 tile, or a CTA pair per 256 x 256 tile (m0 = 128 / 256);
//   * blockNum: how many SMs take part (tiny problems finish sooner on fewer, fuller waves).
// The model is a roofline with the overheads measured on this hardware: tile quantisation
// (waves), the efficiency of the main loop against the sustained cuBLAS rate, an epilogue term
// for short K, launch latency, and the part of the NVLink time that the overlap does not hide.
// Constants were fitted to the benchmark configurations at 1, 2, 4 and 8 GPUs; the CPU test-suite
// checks the model against those measurements.
#ifndef CATCCOS_HOST_COST_MODEL_H
#define CATCCOS_HOST_COST_MODEL_H

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

#include "info.h"

struct COCMatMulInfo {          // utils/info.h:116-121
    int64_t m;
    int64_t k;
    int64_t n;
};

enum class CostModelStatus { SUCCESS, UNSUPPORTED, INVALID_ARGUMENT, NO_VALID_CANDIDATE };

struct CostModelHardwareConfig {
    uint32_t smCount = 148;
    double tensorTflops = 1424.4;        // sustained cuBLAS bf16 of a B200 under its 1 kW power cap (fp8: x2); override with measured figures
    double nvlinkGBs = 770.0;            // peer copy, one direction
    double pairEfficiency = 0.86;        // main loop of the CTA-pair kernels against tensorTflops (long K)
    double oneCtaEfficiency = 0.78;      // ... of the one-CTA kernels (L2 feed: 48 instead of 32 KiB per K-step)
    double mxEfficiency = 0.85;          // MXFP8 main loop against 2 x tensorTflops, before its exposed epilogues
    double launchUs = 8.0;               // launch + pipeline fill + teardown
    double pairSyncUs = 2.0;             // cluster start-up and the pair's cross-CTA barriers
    double epilogueUs = 2.2;             // drain of one 128 x 256 accumulator half (hidden behind the next tile if it is longer)
    double flagRoundTripUs = 10.0;       // a flag that follows data over NVLink, under load
    double exposedCommBase = 0.65;       // fraction of the NVLink time left exposed: base - slope / ranks
    double exposedCommSlope = 1.00;
    double skewPerRank = 0.01;           // the slowest of R GPUs sets the pace: compute x (1 + skew (R - 1))
    double reduceOverhead = 0.12;        // reduce-scatter family with peers: staging writes and partial reads in the epilogue
};

struct CostModelTiling {
    uint32_t m0 = 0, k0 = 0, n0 = 0;     // m0 = 256: CTA pairs, 128: one CTA per tile
    uint32_t blockNum = 0;               // SMs to use (the launchers' blockNum argument)
};

struct CostModelConfig {
    std::vector<uint32_t> m0List{128, 256};
    std::vector<uint32_t> blockNumList{};            // empty: {smCount, smCount / 2, smCount / 4}
    CocDataType dataType = BF16;
    CostModelHardwareConfig hardware{};
};

struct CostModelResult {
    CostModelTiling tiling{};
    double cost = std::numeric_limits<double>::max();        // microseconds
    double computeUs = 0, commUs = 0;                        // its two roofline terms
    CostModelStatus status = CostModelStatus::UNSUPPORTED;
    bool IsSuccess() const { return status == CostModelStatus::SUCCESS; }
};

namespace catccos_cost {

enum class Family { ALLGATHER, REDUCE_SCATTER, ALLREDUCE };

inline bool FamilyOf(CocCommType type, Family &family, bool &mx) {
    mx = false;
    switch (type) {
        case ALLGATHER_MATMUL:
        case ASCEND950_ALLGATHER_MATMUL: family = Family::ALLGATHER; return true;
        case ASCEND950_FP8_MX_ALLGATHER_MATMUL: family = Family::ALLGATHER; mx = true; return true;
        case MATMUL_REDUCE_SCATTER:
        case ASCEND950_MATMUL_REDUCE_SCATTER: family = Family::REDUCE_SCATTER; return true;
        case ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER: family = Family::REDUCE_SCATTER; mx = true; return true;
        case MATMUL_ALLREDUCE: family = Family::ALLREDUCE; return true;
        default: return false;
    }
}

// Time of one candidate.  info carries the reference's meaning of m per operator: rows of one rank
// (AllGather-Matmul) or rows of the full product (ReduceScatter / AllReduce); k is the rank's
// contraction length.
inline CostModelResult Evaluate(const COCMatMulInfo &info, Family family, bool mx, uint32_t rankSize,
                                const CostModelTiling &tiling, const CostModelHardwareConfig &hw) {
    CostModelResult r;
    r.tiling = tiling;
    if (info.m <= 0 || info.n <= 0 || info.k <= 0 || rankSize == 0 || tiling.blockNum == 0 ||
        (tiling.m0 != 128 && tiling.m0 != 256)) {
        r.status = CostModelStatus::INVALID_ARGUMENT;
        return r;
    }
    const bool pair = tiling.m0 == 256;
    if (pair && tiling.blockNum < 2) {
        r.status = CostModelStatus::INVALID_ARGUMENT;
        return r;
    }
    const double R = rankSize;
    // rows every rank multiplies, and how they split into blocks that are tiled separately
    const double blocks = R;                                               // per source (AG) or per owner (RS / AR)
    const double rowsPerBlock = family == Family::ALLGATHER ? static_cast<double>(info.m)
                                                            : std::ceil(static_cast<double>(info.m) / R);
    const double tilesM = std::ceil(rowsPerBlock / tiling.m0);
    const double tilesN = std::ceil(static_cast<double>(info.n) / 256.0);
    const double tiles = blocks * tilesM * tilesN;
    const double units = pair ? std::floor(tiling.blockNum / 2.0) : tiling.blockNum;
    const double waves = std::ceil(tiles / units);
    // one tile on one unit at the main loop's efficiency; a unit is 1 or 2 SMs of hw.smCount
    const double eff = mx ? hw.mxEfficiency : (pair ? hw.pairEfficiency : hw.oneCtaEfficiency);
    const double peak = hw.tensorTflops * (mx ? 2.0 : 1.0) * 1e6;          // flop per microsecond, whole GPU
    const double unitRate = peak * eff * (pair ? 2.0 : 1.0) / hw.smCount;
    const double tileFlops = 2.0 * tiling.m0 * 256.0 * static_cast<double>(info.k);
    const double tileUs = tileFlops / unitRate;
    // the epilogue of a tile overlaps the next tile's main loop (two accumulators; MXFP8 has one)
    const double epi = hw.epilogueUs * (family == Family::ALLGATHER ? 0.6 : 1.0);
    const double exposedEpi = mx ? epi : std::max(0.0, epi - tileUs);
    r.computeUs = waves * (tileUs + exposedEpi) + epi;                      // + the last tile's own epilogue
    if (rankSize > 1) {
        r.computeUs *= 1.0 + hw.skewPerRank * (R - 1);
        if (family != Family::ALLGATHER) r.computeUs *= 1.0 + hw.reduceOverhead;
    }
    // bytes that leave this rank over NVLink
    const double bytesIn = mx ? 1.0 : 2.0, bytesOut = 2.0;
    double commBytes = 0;
    if (family == Family::ALLGATHER)
        commBytes = (R - 1) * static_cast<double>(info.m) * info.k * bytesIn * (mx ? 1.0 + 1.0 / 32 : 1.0);
    else if (family == Family::REDUCE_SCATTER)
        commBytes = (R - 1) / R * static_cast<double>(info.m) * info.n * bytesOut;
    else
        commBytes = 2.0 * (R - 1) / R * static_cast<double>(info.m) * info.n * bytesOut;   // partials out, reduced rows out
    r.commUs = commBytes / (hw.nvlinkGBs * 1e3);
    double cost = hw.launchUs + (pair ? hw.pairSyncUs : 0.0);
    if (rankSize == 1) {
        cost += r.computeUs;
    } else {
        const double exposedFrac = std::max(0.05, hw.exposedCommBase - hw.exposedCommSlope / R);
        // reduce-scatter traffic can only flow while peer tiles are produced: (R-1)/R of the kernel
        const double window = family == Family::ALLGATHER ? 1.0 : (R - 1) / R;
        cost += std::max(r.computeUs, r.commUs / window) + exposedFrac * r.commUs + hw.flagRoundTripUs;
        if (family == Family::ALLREDUCE) cost += 2.0 * hw.flagRoundTripUs;  // second exchange and the copy-out phase
    }
    r.cost = cost;
    r.status = CostModelStatus::SUCCESS;
    return r;
}

inline CostModelResult Select(const COCMatMulInfo &info, Family family, bool mx, uint32_t rankSize,
                              const CostModelConfig &config) {
    CostModelResult best;
    best.status = CostModelStatus::NO_VALID_CANDIDATE;
    const CostModelHardwareConfig &hw = config.hardware;
    std::vector<uint32_t> blocks = config.blockNumList;
    if (blocks.empty()) blocks = {hw.smCount, hw.smCount / 2, hw.smCount / 4};
    for (uint32_t m0 : config.m0List) {
        if (mx && m0 != 256) continue;                 // the MXFP8 operators ship as pair kernels
        for (uint32_t bn : blocks) {
            CostModelTiling t;
            t.m0 = m0;
            t.n0 = 256;
            t.k0 = mx ? 128 : 64;
            t.blockNum = m0 == 256 ? (bn & ~1u) : bn;
            const CostModelResult r = Evaluate(info, family, mx, rankSize, t, hw);
            if (r.status == CostModelStatus::INVALID_ARGUMENT && best.status == CostModelStatus::NO_VALID_CANDIDATE &&
                (info.m <= 0 || info.n <= 0 || info.k <= 0 || rankSize == 0)) {
                best.status = CostModelStatus::INVALID_ARGUMENT;
                return best;
            }
            // ties go to the candidate that keeps more SMs busy with fewer, larger tiles (listed first)
            if (r.IsSuccess() && r.cost < best.cost * (1.0 - 1e-9)) best = r;
        }
    }
    return best;
}

}  // namespace catccos_cost

inline CostModelResult SelectAllGatherTiling(const COCMatMulInfo &info, uint32_t rankSize,
                                             const CostModelConfig &config = CostModelConfig{}) {
    return catccos_cost::Select(info, catccos_cost::Family::ALLGATHER, false, rankSize, config);
}
inline CostModelResult SelectReduceScatterTiling(const COCMatMulInfo &info, uint32_t rankSize,
                                                 const CostModelConfig &config = CostModelConfig{}) {
    return catccos_cost::Select(info, catccos_cost::Family::REDUCE_SCATTER, false, rankSize, config);
}
inline CostModelResult SelectAllReduceTiling(const COCMatMulInfo &info, uint32_t rankSize,
                                             const CostModelConfig &config = CostModelConfig{}) {
    return catccos_cost::Select(info, catccos_cost::Family::ALLREDUCE, false, rankSize, config);
}
inline CostModelResult SelectCostModelTiling(const COCMatMulInfo &info, CocCommType type, uint32_t rankSize,
                                             const CostModelConfig &config = CostModelConfig{}) {
    catccos_cost::Family family;
    bool mx;
    if (!catccos_cost::FamilyOf(type, family, mx)) return CostModelResult{};      // status UNSUPPORTED
    return catccos_cost::Select(info, family, mx, rankSize, config);
}
// Fills the tile fields of `tiling` (m0, n0, k0) from the best candidate; `blockNum`, when given, receives the
// SM count to pass to the launcher.  False (tiling untouched) when the operator has no model.
inline bool ApplyCostModel(const COCMatMulInfo &info, CocCommType type, uint32_t rankSize, CocTilingParams &tiling,
                           const CostModelConfig &config = CostModelConfig{}, uint32_t *blockNum = nullptr) {
    const CostModelResult r = SelectCostModelTiling(info, type, rankSize, config);
    if (!r.IsSuccess()) return false;
    tiling.m0 = r.tiling.m0;
    tiling.n0 = r.tiling.n0;
    tiling.k0 = r.tiling.k0;
    if (blockNum) *blockNum = r.tiling.blockNum;
    return true;
}

#endif  // CATCCOS_HOST_COST_MODEL_H
