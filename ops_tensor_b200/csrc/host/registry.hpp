// Solution registries: where operator implementations plug into the host API.
//
// The flow is the reference's (lib/elementwise/elementwise.hpp:38-71, :204-233, :240-359, :377-393): an
// implementation is an object with a key and an execute function, registered into a process-wide singleton by a
// file-scope registrar object during static initialisation of the shared library; lookup tries the exact key
// first and then the generic one (numModes == 0).  The contraction registry repeats the pattern with a key made
// of operand types and scale modes.
#pragma once

#include <cstdint>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "acl/acl.h"
#include "cann_ops_tensor_types.h"
#include "objects.hpp"

namespace acltensor {

// ------------------------------------------------------------------------------------------------ elementwise

struct SolutionUid {
    acltensorOperator_t op;
    acltensorDataType_t dataType;
    uint32_t numModes;             // 0 = any rank
    OperationType operationType;
    bool operator==(const SolutionUid& o) const {
        return op == o.op && dataType == o.dataType && numModes == o.numModes && operationType == o.operationType;
    }
};

struct SolutionUidHash {
    size_t operator()(const SolutionUid& u) const {
        size_t h = static_cast<size_t>(u.op);
        h = h * 1000003u ^ static_cast<size_t>(u.dataType);
        h = h * 1000003u ^ static_cast<size_t>(u.numModes);
        h = h * 1000003u ^ static_cast<size_t>(u.operationType);
        return h;
    }
};

// Everything an elementwise implementation needs for one call (cf. ElementwiseArgs, elementwise.hpp:76-121).
struct ElementwiseArgs {
    const void* bufferA = nullptr;
    const int64_t* lengthsA = nullptr;
    const int64_t* stridesA = nullptr;
    const int32_t* modesA = nullptr;
    uint32_t numModesA = 0;
    acltensorDataType_t dataTypeA = ACLTENSOR_R_32F;

    const void* bufferC = nullptr;
    const int64_t* lengthsC = nullptr;
    const int64_t* stridesC = nullptr;
    const int32_t* modesC = nullptr;
    uint32_t numModesC = 0;
    acltensorDataType_t dataTypeC = ACLTENSOR_R_32F;

    void* bufferD = nullptr;
    const int64_t* lengthsD = nullptr;
    const int64_t* stridesD = nullptr;
    const int32_t* modesD = nullptr;
    uint32_t numModesD = 0;
    acltensorDataType_t dataTypeD = ACLTENSOR_R_32F;

    const void* alpha = nullptr;
    const void* gamma = nullptr;
    acltensorOperator_t opAC = ACLTENSOR_OP_ADD;
    aclrtStream stream = nullptr;
    void* workspace = nullptr;
};

using ElementwiseBinaryExecuteFunc = acltensorStatus_t (*)(const ElementwiseArgs& args);

class ElementwiseSolution {
public:
    ElementwiseSolution(const SolutionUid& uid, ElementwiseBinaryExecuteFunc fn) : uid_(uid), fn_(fn) {}
    virtual ~ElementwiseSolution() = default;
    const SolutionUid& getUid() const { return uid_; }
    size_t getWorkspaceSize() const { return 0; }
    virtual acltensorStatus_t execute(const ElementwiseArgs& args) const {
        return fn_ ? fn_(args) : ACLTENSOR_STATUS_INTERNAL_ERROR;
    }

private:
    SolutionUid uid_;
    ElementwiseBinaryExecuteFunc fn_;
};

template <class Uid, class Hash, class Solution>
class Registry {
public:
    void registerSolution(std::shared_ptr<Solution> s) {
        if (!s) return;
        std::lock_guard<std::mutex> lock(mutex_);
        table_[s->getUid()] = std::move(s);
    }
    std::shared_ptr<Solution> find(const Uid& uid) const {
        std::lock_guard<std::mutex> lock(mutex_);
        auto it = table_.find(uid);
        return it == table_.end() ? nullptr : it->second;
    }
    size_t size() const {
        std::lock_guard<std::mutex> lock(mutex_);
        return table_.size();
    }

private:
    mutable std::mutex mutex_;
    std::unordered_map<Uid, std::shared_ptr<Solution>, Hash> table_;
};

class ElementwiseSolutionRegistry : public Registry<SolutionUid, SolutionUidHash, ElementwiseSolution> {
public:
    static ElementwiseSolutionRegistry& instance() {
        static ElementwiseSolutionRegistry r;
        return r;
    }
    // exact rank first, then the rank-agnostic entry
    std::vector<std::shared_ptr<ElementwiseSolution>> getSolutions(acltensorOperator_t op, acltensorDataType_t dt,
                                                                   uint32_t numModes, OperationType type) const {
        std::vector<std::shared_ptr<ElementwiseSolution>> out;
        if (auto s = find(SolutionUid{op, dt, numModes, type})) out.push_back(s);
        if (out.empty())
            if (auto s = find(SolutionUid{op, dt, 0, type})) out.push_back(s);
        return out;
    }
};

#define REGISTER_ELEMENTWISE_SOLUTION(OP_NAME, DATA_TYPE, NUM_MODES, OP_TYPE, EXECUTE_FUNC)                         \
    namespace {                                                                                                     \
    struct OP_NAME##_##DATA_TYPE##_##OP_TYPE##_Registrar {                                                          \
        OP_NAME##_##DATA_TYPE##_##OP_TYPE##_Registrar() {                                                           \
            acltensor::SolutionUid uid{ACLTENSOR_OP_##OP_NAME, ACLTENSOR_##DATA_TYPE, NUM_MODES,                    \
                                       acltensor::OperationType::ELEMENTWISE_##OP_TYPE};                            \
            acltensor::ElementwiseSolutionRegistry::instance().registerSolution(                                    \
                std::make_shared<acltensor::ElementwiseSolution>(uid, EXECUTE_FUNC));                               \
        }                                                                                                           \
    };                                                                                                              \
    static OP_NAME##_##DATA_TYPE##_##OP_TYPE##_Registrar g_registrar_##OP_NAME##_##DATA_TYPE##_##OP_TYPE;           \
    }

// ------------------------------------------------------------------------------------------------ contraction

struct ContractionUid {
    acltensorDataType_t dataTypeA;
    acltensorDataType_t dataTypeB;
    int32_t scaleModeA;
    int32_t scaleModeB;
    uint32_t numModesB;            // 2 = dense, 3 = grouped, 0 = either
    bool operator==(const ContractionUid& o) const {
        return dataTypeA == o.dataTypeA && dataTypeB == o.dataTypeB && scaleModeA == o.scaleModeA &&
               scaleModeB == o.scaleModeB && numModesB == o.numModesB;
    }
};

struct ContractionUidHash {
    size_t operator()(const ContractionUid& u) const {
        size_t h = static_cast<size_t>(u.dataTypeA);
        h = h * 1000003u ^ static_cast<size_t>(u.dataTypeB);
        h = h * 1000003u ^ static_cast<size_t>(u.scaleModeA);
        h = h * 1000003u ^ static_cast<size_t>(u.scaleModeB);
        h = h * 1000003u ^ static_cast<size_t>(u.numModesB);
        return h;
    }
};

struct ContractionArgs {
    const acltensorOperationDescriptor* op = nullptr;
    int32_t splitPolicy = ACLTENSOR_SPLIT_AUTO;
    const void* A = nullptr;
    const void* B = nullptr;
    const void* C = nullptr;       // residual or nullptr
    void* D = nullptr;
    const void* scaleA = nullptr;
    const void* scaleB = nullptr;
    const void* bias = nullptr;
    const void* groupList = nullptr;
    void* scaleD = nullptr;
    void* workspace = nullptr;
    uint64_t workspaceSize = 0;
    bool reuseBPrepass = false;
    aclrtStream stream = nullptr;
};

using ContractionWorkspaceFunc = acltensorStatus_t (*)(const acltensorOperationDescriptor& op, int32_t splitPolicy,
                                                       uint64_t* bytes);
using ContractionExecuteFunc = acltensorStatus_t (*)(const ContractionArgs& args);

class ContractionSolution {
public:
    ContractionSolution(const ContractionUid& uid, ContractionWorkspaceFunc ws, ContractionExecuteFunc ex)
        : uid_(uid), ws_(ws), ex_(ex) {}
    const ContractionUid& getUid() const { return uid_; }
    acltensorStatus_t workspaceSize(const acltensorOperationDescriptor& op, int32_t splitPolicy, uint64_t* bytes) const {
        return ws_ ? ws_(op, splitPolicy, bytes) : ACLTENSOR_STATUS_INTERNAL_ERROR;
    }
    acltensorStatus_t execute(const ContractionArgs& args) const {
        return ex_ ? ex_(args) : ACLTENSOR_STATUS_INTERNAL_ERROR;
    }

private:
    ContractionUid uid_;
    ContractionWorkspaceFunc ws_;
    ContractionExecuteFunc ex_;
};

class ContractionSolutionRegistry : public Registry<ContractionUid, ContractionUidHash, ContractionSolution> {
public:
    static ContractionSolutionRegistry& instance() {
        static ContractionSolutionRegistry r;
        return r;
    }
    std::shared_ptr<ContractionSolution> getSolution(ContractionUid uid) const {
        if (auto s = find(uid)) return s;
        uid.numModesB = 0;
        return find(uid);
    }
};

#define REGISTER_CONTRACTION_SOLUTION(NAME, DT_A, DT_B, SCALE_A, SCALE_B, NUM_MODES_B, WORKSPACE_FUNC, EXECUTE_FUNC) \
    namespace {                                                                                                      \
    struct NAME##_ContractionRegistrar {                                                                             \
        NAME##_ContractionRegistrar() {                                                                              \
            acltensor::ContractionUid uid{ACLTENSOR_##DT_A, ACLTENSOR_##DT_B, ACLTENSOR_SCALE_##SCALE_A,             \
                                          ACLTENSOR_SCALE_##SCALE_B, NUM_MODES_B};                                   \
            acltensor::ContractionSolutionRegistry::instance().registerSolution(                                     \
                std::make_shared<acltensor::ContractionSolution>(uid, WORKSPACE_FUNC, EXECUTE_FUNC));                \
        }                                                                                                            \
    };                                                                                                               \
    static NAME##_ContractionRegistrar g_contraction_registrar_##NAME;                                               \
    }

}  // namespace acltensor
