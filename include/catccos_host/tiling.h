// Enumeration of the tiling candidates of an operator and the CSV the tiling search writes — the
// counterpart of the reference's tests/dynamic_tiling/include/tiling.h (search space :21-26,
// GetTilings :60-92, CreateTilingFile :94-107, WriteTilingInfos :109-127).  The reference's axes
// (commInterval, commTileM, commNpuSplit, commDataSplit) do not exist on B200 (see cost_model.h);
// the candidates here are tile x SMs used, each with the cost model's prediction so that a search
// run can be compared against it.
#ifndef CATCCOS_HOST_TILING_H
#define CATCCOS_HOST_TILING_H

#include <cerrno>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "cost_model.h"
#include "operator_registry.h"

const std::vector<uint32_t> vM0 = {128, 256};                       // one CTA per tile / CTA pair per tile
const std::vector<uint32_t> vBlockNumDivisor = {1, 2, 4};           // all SMs, half, a quarter

struct TilingCandidate {
    CocTilingParams tiling;
    uint32_t blockNum;
    double modelUs;          // the cost model's prediction; < 0 when the operator has no model
};

// Every candidate the operator's own CheckCocTilingParams accepts.
inline void GetTilings(std::vector<TilingCandidate> &out, CocTilingParams t, const std::string &opName, int rankSize,
                       const CostModelHardwareConfig &hw = CostModelHardwareConfig{}) {
    auto op = OperatorRegistry::Instance().CreateOperator(opName);
    if (!op) {
        std::cout << "Operator " << opName << " not found!" << std::endl;
        return;
    }
    t.rankSize = static_cast<uint32_t>(rankSize);
    const CocCommType type = op->GetActualKernelType(t);
    catccos_cost::Family family;
    bool mx = false;
    const bool modelled = catccos_cost::FamilyOf(type, family, mx);
    for (uint32_t m0 : vM0) {
        if (mx && m0 != 256) continue;                              // the MXFP8 operators exist as pair kernels only
        for (uint32_t div : vBlockNumDivisor) {
            TilingCandidate c;
            c.tiling = t;
            c.tiling.m0 = m0;
            c.tiling.n0 = 256;
            c.tiling.k0 = mx ? 128 : 64;
            c.blockNum = hw.smCount / div;
            if (m0 == 256) c.blockNum &= ~1u;
            if (c.blockNum == 0 || !op->CheckCocTilingParams(static_cast<uint32_t>(rankSize), c.tiling)) continue;
            c.modelUs = -1.0;
            if (modelled) {
                CostModelTiling ct;
                ct.m0 = m0;
                ct.n0 = 256;
                ct.k0 = c.tiling.k0;
                ct.blockNum = c.blockNum;
                const COCMatMulInfo info{t.m, t.k, t.n};
                const CostModelResult r = catccos_cost::Evaluate(info, family, mx, static_cast<uint32_t>(rankSize), ct, hw);
                if (r.IsSuccess()) c.modelUs = r.cost;
            }
            out.push_back(c);
        }
    }
}

inline bool CreateTilingFile(const std::string &filename) {
    std::ofstream outFile(filename, std::ios::out);
    if (!outFile.is_open()) {
        std::cerr << "Open file failed." << std::endl;
        return false;
    }
    outFile << "Op,M,K,N,Transpose A,Transpose B,M0,N0,K0,blockNum,Model(us),Time(us)\n";
    return true;
}

// Appends one row per candidate; the last column is left for the measured time, as in the reference.
inline bool WriteTilingInfos(const std::string &opName, const std::vector<TilingCandidate> &candidates,
                             const std::string &filename, int transA = 0, int transB = 1) {
    std::ofstream f(filename, std::ios::out | std::ios::app);
    if (!f) {
        std::cerr << "Open file failed. path = " << filename << ", error = " << std::strerror(errno) << std::endl;
        return false;
    }
    for (const TilingCandidate &c : candidates) {
        f << opName << "," << c.tiling.m << "," << c.tiling.k << "," << c.tiling.n << "," << transA << "," << transB << ","
          << c.tiling.m0 << "," << c.tiling.n0 << "," << c.tiling.k0 << "," << c.blockNum << ",";
        if (c.modelUs >= 0) f << c.modelUs;
        f << ",\n";
    }
    return true;
}

#endif  // CATCCOS_HOST_TILING_H
