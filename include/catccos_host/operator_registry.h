// Name -> factory registry with static-initialisation registration (utils/operator_registry.h:26-68).
#ifndef CATCCOS_HOST_OPERATOR_REGISTRY_H
#define CATCCOS_HOST_OPERATOR_REGISTRY_H

#include <mutex>
#include <unordered_map>
#include <vector>

#include "catccos_operator.h"

class OperatorRegistry {
public:
    static OperatorRegistry &Instance() {
        static OperatorRegistry instance;
        return instance;
    }
    // false when the name is already taken (the first registration wins)
    bool RegisterOperator(const std::string &opType, OperatorCreator creator) {
        std::lock_guard<std::mutex> lock(mutex_);
        return registry_.emplace(opType, std::move(creator)).second;
    }
    // nullptr for an unknown name
    std::unique_ptr<CatccosOperator> CreateOperator(const std::string &opType) {
        std::lock_guard<std::mutex> lock(mutex_);
        const auto it = registry_.find(opType);
        return it == registry_.end() ? nullptr : it->second();
    }
    std::vector<std::string> Names() {
        std::lock_guard<std::mutex> lock(mutex_);
        std::vector<std::string> out;
        for (const auto &kv : registry_) out.push_back(kv.first);
        return out;
    }

private:
    std::unordered_map<std::string, OperatorCreator> registry_;
    std::mutex mutex_;
};

#define REGISTER_OPERATOR(op_type, op_class)                                                             \
    namespace {                                                                                          \
    struct op_class##_registrar {                                                                        \
        op_class##_registrar() {                                                                         \
            OperatorRegistry::Instance().RegisterOperator(                                               \
                op_type, []() -> std::unique_ptr<CatccosOperator> { return std::make_unique<op_class>(); }); \
        }                                                                                                \
    };                                                                                                   \
    static op_class##_registrar op_class##_instance;                                                     \
    }

#endif  // CATCCOS_HOST_OPERATOR_REGISTRY_H
