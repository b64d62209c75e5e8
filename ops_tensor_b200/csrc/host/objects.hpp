// Host-side objects behind the opaque acltensor* handles.
//
// They play the roles of the reference's lib/core structs (handle.hpp:71-74, tensor_descriptor.hpp:28-92,
// operation_descriptor.hpp:40-84, plan_preference.hpp:33-45, plan.hpp:36-48) with the same ownership rules:
// an operation descriptor points at, and does not own, its tensor descriptors; a plan points at, and does not own,
// its operation descriptor and preference; the chosen solution is cached in the preference as a shared_ptr.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "cann_ops_tensor_types.h"

namespace acltensor {

enum class OperationType : uint32_t {
    ELEMENTWISE_BINARY = 0,
    ELEMENTWISE_TRINARY = 1,   // reserved by the reference, not implemented there or here
    CONTRACTION = 2,
};

// Size of one element in bits (4 for packed E2M1); 0 for a type this build does not know.
inline uint32_t DataTypeBits(acltensorDataType_t t) {
    switch (t) {
        case ACLTENSOR_R_16F: case ACLTENSOR_R_16BF: return 16;
        case ACLTENSOR_R_32F: case ACLTENSOR_R_32I: case ACLTENSOR_R_32U: return 32;
        case ACLTENSOR_R_64F: case ACLTENSOR_R_64I: case ACLTENSOR_C_32F: return 64;
        case ACLTENSOR_C_64F: return 128;
        case ACLTENSOR_R_8I: case ACLTENSOR_R_8U: case ACLTENSOR_R_8F_E4M3: case ACLTENSOR_R_8F_E5M2:
        case ACLTENSOR_R_8F_UE8M0: return 8;
        case ACLTENSOR_R_4F_E2M1: return 4;
        default: return 0;
    }
}

// Byte size for whole-byte types (the reference's GetDataTypeSize, lib/utils/type_utils.hpp:29-58); 0 for sub-byte.
inline size_t GetDataTypeSize(acltensorDataType_t t) { return DataTypeBits(t) / 8; }

// Types a tensor descriptor may carry in this build.  The reference accepts FP32 only
// (lib/core/tensor_descriptor.cpp:43-45); the contraction path adds its operand, scale, output and index types.
inline bool IsDescriptorTypeSupported(acltensorDataType_t t) {
    switch (t) {
        case ACLTENSOR_R_32F: case ACLTENSOR_R_16BF: case ACLTENSOR_R_16F: case ACLTENSOR_R_8F_E4M3:
        case ACLTENSOR_R_8F_E5M2: case ACLTENSOR_R_4F_E2M1:
        case ACLTENSOR_R_8F_UE8M0: case ACLTENSOR_R_8U: case ACLTENSOR_R_64I:
        case ACLTENSOR_R_8I: case ACLTENSOR_R_32I:          // INT8 operands and their int32 sums / bias
            return true;
        default:
            return false;
    }
}

acltensorStatus_t CheckOperator(acltensorOperator_t op);
acltensorStatus_t CheckComputeDescriptor(acltensorComputeDescriptor_t desc);

}  // namespace acltensor

namespace acltensor {

// What a contraction plan may choose when the caller left it open: tile width, 1- or 2-CTA tiles, scheduler mode.
struct PlanChoice {
    int32_t tileN = 0, ctaPair = 0, splitPolicy = ACLTENSOR_SPLIT_AUTO;
};

// The handle's plan cache (the reference reserves acltensorHandleResizePlanCache / WritePlanCacheToFile /
// ReadPlanCacheFromFile for it, lib/core/handle.cpp:105-108): problem signature -> choice, oldest entry evicted first.
class PlanCache {
public:
    bool find(const std::string& key, PlanChoice* out) {
        std::lock_guard<std::mutex> lock(m_);
        for (const auto& e : entries_)
            if (e.first == key) { *out = e.second; return true; }
        return false;
    }
    void insert(const std::string& key, const PlanChoice& c) {
        std::lock_guard<std::mutex> lock(m_);
        for (auto& e : entries_)
            if (e.first == key) { e.second = c; return; }
        entries_.emplace_back(key, c);
        trim();
    }
    void resize(uint32_t n) {
        std::lock_guard<std::mutex> lock(m_);
        capacity_ = n;
        trim();
    }
    std::vector<std::pair<std::string, PlanChoice>> snapshot() {
        std::lock_guard<std::mutex> lock(m_);
        return entries_;
    }

private:
    void trim() {
        if (entries_.size() > capacity_) entries_.erase(entries_.begin(), entries_.end() - capacity_);
    }
    std::mutex m_;
    uint32_t capacity_ = 64;
    std::vector<std::pair<std::string, PlanChoice>> entries_;
};

}  // namespace acltensor

struct acltensorHandle {
    std::shared_ptr<acltensor::PlanCache> planCache = std::make_shared<acltensor::PlanCache>();
    int32_t deviceId = -1;      // CUDA device current at creation (-1: none visible)
    int32_t smCount = 0;
    int32_t ccMajor = 0, ccMinor = 0;
    char deviceName[64] = {0};
};

struct acltensorTensorDescriptor {
    acltensorDataType_t dataType = ACLTENSOR_R_32F;
    uint32_t numModes = 0;
    std::vector<int64_t> lens;
    std::vector<int64_t> strides;          // in elements
    uint32_t alignmentRequirement = 0;
    uint32_t elementBits = 0;
    size_t elementSize = 0;                // bytes; 0 for sub-byte types
    size_t totalElements = 0;
    size_t totalBytes = 0;
    bool isContiguous = true;

    void finalize();                       // fills strides (when absent) and the derived members
};

struct acltensorOperationDescriptor {
    acltensor::OperationType operationType = acltensor::OperationType::ELEMENTWISE_BINARY;
    acltensorTensorDescriptor_t descA = nullptr, descB = nullptr, descC = nullptr, descD = nullptr;
    std::vector<int32_t> modeA, modeB, modeC, modeD;
    acltensorOperator_t opA = ACLTENSOR_OP_IDENTITY, opB = ACLTENSOR_OP_IDENTITY, opC = ACLTENSOR_OP_IDENTITY;
    acltensorOperator_t opAC = ACLTENSOR_OP_ADD, opAB = ACLTENSOR_OP_ADD, opABC = ACLTENSOR_OP_IDENTITY;
    acltensorComputeDescriptor_t descCompute = ACLTENSOR_COMPUTE_DESC_32F;

    // contraction attributes
    int32_t scaleModeA = ACLTENSOR_SCALE_NONE, scaleModeB = ACLTENSOR_SCALE_NONE;
    int32_t epilogueAct = ACLTENSOR_OP_IDENTITY;
    int32_t biasType = -1;
    int32_t groupCount = 0;
    int32_t splitPolicy = ACLTENSOR_SPLIT_AUTO;
    int32_t tileN = 0;
    int32_t smLimit = 0;
    int32_t bIsStatic = 0;
    int32_t ctaPair = 0;

    // contraction geometry, resolved at creation
    int64_t M = 0, N = 0, K = 0;
    int64_t lda = 0, ldb = 0, ldc = 0, ldd = 0;       // elements
    int64_t groupStrideB = 0;                         // elements between consecutive groups of B
    int32_t batchModes = 0;                           // leading batch modes of D (0..4)
    int32_t batchC[4] = {1, 1, 1, 1}, batchA[4] = {1, 1, 1, 1}, batchB[4] = {1, 1, 1, 1};   // right-aligned extents
    int32_t biasPerBatch = 0;                         // bias is [batches][N] instead of [N]
    int32_t scaleModeD = ACLTENSOR_SCALE_NONE;        // MX_E8M0_VEC32: the epilogue quantises D
    int32_t bNMajor = 0;                              // B is stored [K][N] with N contiguous (ldb = its K stride)

    size_t getTotalElements() const { return descD ? descD->totalElements : 0; }
    acltensorDataType_t getDataType() const { return descD ? descD->dataType : ACLTENSOR_R_32F; }
};

struct acltensorPlanPreference {
    acltensorAlgo_t algo = ACLTENSOR_ALGO_DEFAULT;
    std::vector<void*> candidates;
    std::shared_ptr<void> solution;       // chosen at first execute (elementwise) or at plan creation (contraction)
};

struct acltensorPlan {
    acltensorOperationDescriptor_t opDesc = nullptr;
    acltensorPlanPreference_t pref = nullptr;
    uint64_t requiredWorkspace = 0;
    // contraction plans
    std::shared_ptr<void> solution;
    int32_t splitPolicy = ACLTENSOR_SPLIT_AUTO;   // policy after the workspace limit was applied
    const void* preparedB = nullptr;              // B / scaleB / workspace whose pre-pass results are still valid
    const void* preparedScaleB = nullptr;
    const void* preparedWorkspace = nullptr;
    uint64_t stamp = 0;                           // unique per plan, given at its first contraction call (0 = none yet)
    // A choice taken from the handle's plan cache or found by timing (ALGO_DEFAULT_PATIENT) lives in a private copy of
    // the operation descriptor with tile width and CTA pairing filled in; the caller's descriptor stays as it is.
    std::unique_ptr<acltensorOperationDescriptor> tunedOp;
    acltensor::PlanChoice choice;                 // what the plan runs with (0 / AUTO = left to the launch layer)
    std::shared_ptr<acltensor::PlanCache> cache;  // the creating handle's cache (outlives the handle if need be)
    std::string cacheKey;                         // empty: the caller fixed the choice, nothing to cache
    bool needsTuning = false;                     // PATIENT plan that has not timed its candidates yet

    size_t getTotalElements() const { return opDesc ? opDesc->getTotalElements() : 0; }
};
