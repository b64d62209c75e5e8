// Handle, tensor descriptor, operation descriptor, plan preference, plan, error strings and version: the object
// management half of the host API.  Behaviour per entry point follows the reference implementation cited beside
// each function; the code is new.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <new>
#include <sstream>

#include "blaze_b200.h"
#include "cann_ops_tensor.h"
#include "objects.hpp"
#include "registry.hpp"

namespace acltensor {

// The reference accepts IDENTITY and ADD only (lib/utils/validation.cpp:26-38).
acltensorStatus_t CheckOperator(acltensorOperator_t op) {
    return (op == ACLTENSOR_OP_IDENTITY || op == ACLTENSOR_OP_ADD) ? ACLTENSOR_STATUS_SUCCESS
                                                                   : ACLTENSOR_STATUS_NOT_SUPPORTED;
}

// NONE is an invalid argument, anything but 32F is unsupported (lib/utils/validation.cpp:47-64).
acltensorStatus_t CheckComputeDescriptor(acltensorComputeDescriptor_t desc) {
    if (desc == ACLTENSOR_COMPUTE_DESC_NONE) return ACLTENSOR_STATUS_INVALID_VALUE;
    return desc == ACLTENSOR_COMPUTE_DESC_32F ? ACLTENSOR_STATUS_SUCCESS : ACLTENSOR_STATUS_NOT_SUPPORTED;
}

}  // namespace acltensor

void acltensorTensorDescriptor::finalize() {
    elementBits = acltensor::DataTypeBits(dataType);
    elementSize = elementBits / 8;
    totalElements = 1;
    for (uint32_t i = 0; i < numModes; ++i) totalElements *= static_cast<size_t>(lens[i]);
    if (strides.size() != numModes) {
        strides.assign(numModes, 1);
        for (int32_t i = static_cast<int32_t>(numModes) - 2; i >= 0; --i) strides[i] = strides[i + 1] * lens[i + 1];
        isContiguous = true;
    } else {
        isContiguous = true;
        int64_t expect = 1;
        for (int32_t i = static_cast<int32_t>(numModes) - 1; i >= 0; --i) {
            if (strides[i] != expect) { isContiguous = false; break; }
            expect *= lens[i];
        }
    }
    totalBytes = (totalElements * elementBits + 7) / 8;
}

// ------------------------------------------------------------------------------------------------ handle
// reference: lib/core/handle.cpp:75-103 (creation never fails for lack of a device; destroy accepts NULL)

acltensorStatus_t acltensorCreate(acltensorHandle_t* handle) {
    if (handle == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    acltensorHandle* h = new (std::nothrow) acltensorHandle();
    if (h == nullptr) return ACLTENSOR_STATUS_ALLOC_FAILED;
    int32_t sms = 0, major = 0, minor = 0;
    int32_t device = -1;
    if (blazeDeviceInfo(&sms, &major, &minor) == ACLTENSOR_STATUS_SUCCESS &&
        blazeCurrentDevice(&device) == ACLTENSOR_STATUS_SUCCESS) {
        h->deviceId = device;               // the handle belongs to the device that is current now
        h->smCount = sms;
        h->ccMajor = major;
        h->ccMinor = minor;
        std::strncpy(h->deviceName, (major == 10) ? "B200-class (sm_100)" : "unsupported CUDA device",
                     sizeof(h->deviceName) - 1);
    }
    *handle = h;
    return ACLTENSOR_STATUS_SUCCESS;
}

acltensorStatus_t acltensorDestroy(acltensorHandle_t handle) {
    delete handle;
    return ACLTENSOR_STATUS_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ plan cache
// The three entry points the reference reserves (lib/core/handle.cpp:105-108, docs/implementation.md:62-64).  The
// file is text: a header line, then "<problem signature> <tileN> <ctaPair> <splitPolicy>" per entry, oldest first.

static const char kPlanCacheMagic[] = "acltensor-plan-cache 1";

acltensorStatus_t acltensorHandleResizePlanCache(acltensorHandle_t handle, const uint32_t numEntries) {
    if (handle == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    handle->planCache->resize(numEntries);
    return ACLTENSOR_STATUS_SUCCESS;
}

acltensorStatus_t acltensorHandleWritePlanCacheToFile(const acltensorHandle_t handle, const char filename[]) {
    if (handle == nullptr || filename == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    std::ofstream f(filename, std::ios::trunc);
    if (!f) return ACLTENSOR_STATUS_IO_ERROR;
    f << kPlanCacheMagic << "\n";
    for (const auto& e : handle->planCache->snapshot())
        f << e.first << ' ' << e.second.tileN << ' ' << e.second.ctaPair << ' ' << e.second.splitPolicy << "\n";
    f.flush();
    return f ? ACLTENSOR_STATUS_SUCCESS : ACLTENSOR_STATUS_IO_ERROR;
}

acltensorStatus_t acltensorHandleReadPlanCacheFromFile(acltensorHandle_t handle, const char filename[],
                                                       uint32_t* numCachelinesRead) {
    if (handle == nullptr || filename == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (numCachelinesRead) *numCachelinesRead = 0;
    std::ifstream f(filename);
    if (!f) return ACLTENSOR_STATUS_IO_ERROR;
    std::string line;
    if (!std::getline(f, line) || line != kPlanCacheMagic) return ACLTENSOR_STATUS_INVALID_VALUE;
    // parse everything before touching the cache: a damaged file changes nothing
    std::vector<std::pair<std::string, acltensor::PlanChoice>> entries;
    while (std::getline(f, line)) {
        if (line.empty()) continue;
        std::istringstream in(line);
        std::string key, rest;
        acltensor::PlanChoice c;
        if (!(in >> key >> c.tileN >> c.ctaPair >> c.splitPolicy) || (in >> rest)) return ACLTENSOR_STATUS_INVALID_VALUE;
        const bool tile_ok = c.tileN == 0 || c.tileN == 128 || c.tileN == 224 || c.tileN == 256;
        if (!tile_ok || c.ctaPair < 0 || c.ctaPair > 2 || c.splitPolicy < ACLTENSOR_SPLIT_AUTO ||
            c.splitPolicy > ACLTENSOR_SPLIT_STREAM_K)
            return ACLTENSOR_STATUS_INVALID_VALUE;
        entries.emplace_back(key, c);
    }
    for (const auto& e : entries) handle->planCache->insert(e.first, e.second);
    if (numCachelinesRead) *numCachelinesRead = static_cast<uint32_t>(entries.size());
    return ACLTENSOR_STATUS_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ tensor descriptor
// reference: lib/core/tensor_descriptor.cpp:23-81

acltensorStatus_t acltensorCreateTensorDescriptor(const acltensorHandle_t handle, acltensorTensorDescriptor_t* desc,
                                                  const uint32_t rank, const int64_t dimSizes[],
                                                  const int64_t stridesIn[], acltensorDataType_t dType,
                                                  uint32_t alignReq) {
    (void)handle;
    if (desc == nullptr || dimSizes == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (rank == 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (!acltensor::IsDescriptorTypeSupported(dType)) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    for (uint32_t i = 0; i < rank; ++i)
        if (dimSizes[i] < 0) return ACLTENSOR_STATUS_INVALID_VALUE;
    acltensorTensorDescriptor* d = new (std::nothrow) acltensorTensorDescriptor();
    if (d == nullptr) return ACLTENSOR_STATUS_ALLOC_FAILED;
    d->dataType = dType;
    d->numModes = rank;
    d->alignmentRequirement = alignReq;
    d->lens.assign(dimSizes, dimSizes + rank);
    if (stridesIn != nullptr) d->strides.assign(stridesIn, stridesIn + rank);
    d->finalize();
    *desc = d;
    return ACLTENSOR_STATUS_SUCCESS;
}

acltensorStatus_t acltensorDestroyTensorDescriptor(acltensorTensorDescriptor_t desc) {
    delete desc;
    return ACLTENSOR_STATUS_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ elementwise descriptor
// reference: lib/core/operation_descriptor.cpp:123-181 (argument checks, then operators, then compute type)

acltensorStatus_t acltensorCreateElementwiseBinary(const acltensorHandle_t handle, acltensorOperationDescriptor_t* desc,
                                                   const acltensorTensorDescriptor_t descA, const int32_t modeA[],
                                                   acltensorOperator_t opA, const acltensorTensorDescriptor_t descC,
                                                   const int32_t modeC[], acltensorOperator_t opC,
                                                   const acltensorTensorDescriptor_t descD, const int32_t modeD[],
                                                   acltensorOperator_t opAC,
                                                   const acltensorComputeDescriptor_t descCompute) {
    (void)handle;
    if (desc == nullptr || descA == nullptr || descC == nullptr || descD == nullptr)
        return ACLTENSOR_STATUS_INVALID_VALUE;
    if (modeA == nullptr || modeC == nullptr || modeD == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    for (acltensorOperator_t op : {opA, opC, opAC}) {
        const acltensorStatus_t st = acltensor::CheckOperator(op);
        if (st != ACLTENSOR_STATUS_SUCCESS) return st;
    }
    const acltensorStatus_t st = acltensor::CheckComputeDescriptor(descCompute);
    if (st != ACLTENSOR_STATUS_SUCCESS) return st;

    acltensorOperationDescriptor* d = new (std::nothrow) acltensorOperationDescriptor();
    if (d == nullptr) return ACLTENSOR_STATUS_ALLOC_FAILED;
    d->operationType = acltensor::OperationType::ELEMENTWISE_BINARY;
    d->descA = descA;
    d->descC = descC;
    d->descD = descD;
    d->modeA.assign(modeA, modeA + descA->numModes);
    d->modeC.assign(modeC, modeC + descC->numModes);
    d->modeD.assign(modeD, modeD + descD->numModes);
    d->opA = opA;
    d->opC = opC;
    d->opAC = opAC;
    d->descCompute = descCompute;
    *desc = d;
    return ACLTENSOR_STATUS_SUCCESS;
}

acltensorStatus_t acltensorDestroyOperationDescriptor(acltensorOperationDescriptor_t desc) {
    delete desc;      // the tensor descriptors belong to the caller
    return ACLTENSOR_STATUS_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ plan preference
// reference: lib/core/plan_preference.cpp:22-56 (ALGO_DEFAULT only; ALGO_DEFAULT_PATIENT is declared in its enum,
// include/cann_ops_tensor_types.h:113, "more exact but slower choice": here a contraction plan times its candidates)

acltensorStatus_t acltensorCreatePlanPreference(const acltensorHandle_t handle, acltensorPlanPreference_t* pref,
                                                acltensorAlgo_t algo) {
    (void)handle;
    if (pref == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (algo != ACLTENSOR_ALGO_DEFAULT && algo != ACLTENSOR_ALGO_DEFAULT_PATIENT) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    acltensorPlanPreference* p = new (std::nothrow) acltensorPlanPreference();
    if (p == nullptr) return ACLTENSOR_STATUS_ALLOC_FAILED;
    p->algo = algo;
    *pref = p;
    return ACLTENSOR_STATUS_SUCCESS;
}

acltensorStatus_t acltensorDestroyPlanPreference(acltensorPlanPreference_t pref) {
    delete pref;
    return ACLTENSOR_STATUS_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ plan
// reference: lib/core/plan.cpp:24-73.  Elementwise plans need no workspace and ignore the limit, as there.
// Contraction plans pick their solution here and apply the limit (see api_contraction.cpp).

namespace acltensor {
acltensorStatus_t FinishContractionPlan(acltensorPlan* plan, uint64_t workspaceSizeLimit, const acltensorHandle* handle);
}

acltensorStatus_t acltensorCreatePlan(const acltensorHandle_t handle, acltensorPlan_t* plan,
                                      const acltensorOperationDescriptor_t desc, const acltensorPlanPreference_t pref,
                                      uint64_t workspaceSizeLimit) {
    if (plan == nullptr || desc == nullptr || pref == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (desc->operationType != acltensor::OperationType::ELEMENTWISE_BINARY &&
        desc->operationType != acltensor::OperationType::CONTRACTION)
        return ACLTENSOR_STATUS_NOT_SUPPORTED;
    acltensorPlan* p = new (std::nothrow) acltensorPlan();
    if (p == nullptr) return ACLTENSOR_STATUS_ALLOC_FAILED;
    p->opDesc = desc;
    p->pref = pref;
    p->requiredWorkspace = 0;
    if (desc->operationType == acltensor::OperationType::CONTRACTION) {
        const acltensorStatus_t st = acltensor::FinishContractionPlan(p, workspaceSizeLimit, handle);
        if (st != ACLTENSOR_STATUS_SUCCESS) {
            delete p;
            return st;
        }
    }
    *plan = p;
    return ACLTENSOR_STATUS_SUCCESS;
}

acltensorStatus_t acltensorDestroyPlan(acltensorPlan_t plan) {
    delete plan;      // operation descriptor and preference belong to the caller
    return ACLTENSOR_STATUS_SUCCESS;
}

acltensorStatus_t acltensorPlanGetKernelChoice(const acltensorPlan_t plan, int32_t* tileN, int32_t* ctaPair,
                                               int32_t* splitPolicy, int32_t* pendingTuning) {
    if (plan == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (tileN) *tileN = plan->choice.tileN;
    if (ctaPair) *ctaPair = plan->choice.ctaPair;
    if (splitPolicy) *splitPolicy = plan->choice.splitPolicy;
    if (pendingTuning) *pendingTuning = plan->needsTuning ? 1 : 0;
    return ACLTENSOR_STATUS_SUCCESS;
}

acltensorStatus_t acltensorPlanGetRequiredWorkspace(const acltensorPlan_t plan, uint64_t* bytes) {
    if (plan == nullptr || bytes == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    *bytes = plan->requiredWorkspace;
    return ACLTENSOR_STATUS_SUCCESS;
}

// ------------------------------------------------------------------------------------------------ utilities
// reference: lib/utils/utils.cpp:21-60 (same strings, version 1.0.0 = 1 << 16)

const char* acltensorGetErrorString(const acltensorStatus_t error) {
    switch (error) {
        case ACLTENSOR_STATUS_SUCCESS: return "The operation completed successfully.";
        case ACLTENSOR_STATUS_NOT_INITIALIZED: return "The library was not initialized.";
        case ACLTENSOR_STATUS_ALLOC_FAILED: return "Memory allocation failed.";
        case ACLTENSOR_STATUS_INVALID_VALUE: return "Invalid parameter value.";
        case ACLTENSOR_STATUS_ARCH_MISMATCH: return "Architecture mismatch.";
        case ACLTENSOR_STATUS_EXECUTION_FAILED: return "Kernel execution failed.";
        case ACLTENSOR_STATUS_INTERNAL_ERROR: return "Internal error.";
        case ACLTENSOR_STATUS_NOT_SUPPORTED: return "Operation not supported.";
        case ACLTENSOR_STATUS_INSUFFICIENT_WORKSPACE: return "Insufficient workspace size.";
        case ACLTENSOR_STATUS_INSUFFICIENT_DRIVER: return "Insufficient driver version.";
        case ACLTENSOR_STATUS_IO_ERROR: return "I/O error.";
        default: return "Unknown error.";
    }
}

size_t acltensorGetVersion(void) { return (1u << 16) | (0u << 8) | 0u; }

acltensorStatus_t acltensorGetDeviceStatus(const acltensorHandle_t handle, int32_t* deviceCode) {
    (void)handle;
    int32_t code = 0;
    const int st = blazeDeviceStatus(&code, 1);
    if (st != ACLTENSOR_STATUS_SUCCESS) return static_cast<acltensorStatus_t>(st);
    if (deviceCode) *deviceCode = code;
    return code == 0 ? ACLTENSOR_STATUS_SUCCESS : ACLTENSOR_STATUS_EXECUTION_FAILED;
}
