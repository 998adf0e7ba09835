// Operator base class of the host layer: same virtuals as utils/catccos_operator.h:31-41.
#ifndef CATCCOS_HOST_OPERATOR_H
#define CATCCOS_HOST_OPERATOR_H

#include <functional>
#include <memory>
#include <string>

#include "info.h"

class CatccosOperator {
public:
    virtual ~CatccosOperator() = default;
    virtual bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams &cocTiling) = 0;
    virtual void AllocateDeviceSpace(KernelParams &params, const CocTilingParams &cocTiling, uint32_t rankId,
                                     std::string dataFile = "") = 0;
    virtual void WriteResultFile(const KernelParams &params, const CocTilingParams &cocTiling, uint32_t rankId,
                                 std::string dataFile = "") = 0;
    virtual size_t GetWorkspaceSize(const CocTilingParams &cocTiling) = 0;
    virtual CocCommType GetActualKernelType(const CocTilingParams &cocTiling) = 0;
};

using OperatorCreator = std::function<std::unique_ptr<CatccosOperator>()>;

#endif  // CATCCOS_HOST_OPERATOR_H
