// acltensorElementwiseBinaryExecute and the one registered elementwise solution (ADD on FP32).
//
// Dispatch follows the reference (lib/elementwise/elementwise_binary.cpp:26-68): validate, pick the solution on
// first use (exact rank, then rank-agnostic), cache it in the preference, build the argument block, execute.  The
// ADD solution mirrors the reference's in what it looks at: alpha and gamma are ignored and only the element count
// of D is used (src/add/add_solution.cpp:217-291).  Unlike the reference it does not synchronise the stream.
#include "blaze_b200.h"
#include "cann_ops_tensor.h"
#include "objects.hpp"
#include "registry.hpp"

using namespace acltensor;

static acltensorStatus_t AddF32Execute(const ElementwiseArgs& args) {
    if (args.bufferA == nullptr || args.bufferC == nullptr || args.bufferD == nullptr)
        return ACLTENSOR_STATUS_INVALID_VALUE;
    int64_t n = 1;
    for (uint32_t i = 0; i < args.numModesD; ++i) n *= args.lengthsD[i];
    return static_cast<acltensorStatus_t>(blazeAddF32(args.bufferA, args.bufferC, args.bufferD, n, args.stream));
}

REGISTER_ELEMENTWISE_SOLUTION(ADD, R_32F, 0, BINARY, AddF32Execute);

acltensorStatus_t acltensorElementwiseBinaryExecute(const acltensorHandle_t handle, const acltensorPlan_t plan,
                                                    const void* alpha, const void* A, const void* gamma,
                                                    const void* C, void* D, aclrtStream stream) {
    (void)handle;
    if (plan == nullptr || A == nullptr || C == nullptr || D == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    acltensorOperationDescriptor* op = plan->opDesc;
    acltensorPlanPreference* pref = plan->pref;
    if (op == nullptr || pref == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;
    if (op->operationType != OperationType::ELEMENTWISE_BINARY) return ACLTENSOR_STATUS_NOT_SUPPORTED;
    if (op->descD == nullptr) return ACLTENSOR_STATUS_INVALID_VALUE;

    std::shared_ptr<ElementwiseSolution> solution;
    if (pref->solution) {
        solution = std::static_pointer_cast<ElementwiseSolution>(pref->solution);
    } else {
        auto found = ElementwiseSolutionRegistry::instance().getSolutions(op->opAC, op->descD->dataType,
                                                                          op->descD->numModes, op->operationType);
        if (found.empty()) return ACLTENSOR_STATUS_NOT_SUPPORTED;
        solution = found.front();
        pref->solution = solution;
    }

    ElementwiseArgs args;
    args.bufferA = A;
    args.bufferC = C;
    args.bufferD = D;
    if (op->descA) {
        args.lengthsA = op->descA->lens.data();
        args.stridesA = op->descA->strides.data();
        args.numModesA = op->descA->numModes;
        args.dataTypeA = op->descA->dataType;
    }
    if (op->descC) {
        args.lengthsC = op->descC->lens.data();
        args.stridesC = op->descC->strides.data();
        args.numModesC = op->descC->numModes;
        args.dataTypeC = op->descC->dataType;
    }
    args.lengthsD = op->descD->lens.data();
    args.stridesD = op->descD->strides.data();
    args.numModesD = op->descD->numModes;
    args.dataTypeD = op->descD->dataType;
    args.modesA = op->modeA.data();
    args.modesC = op->modeC.data();
    args.modesD = op->modeD.data();
    args.alpha = alpha;
    args.gamma = gamma;
    args.opAC = op->opAC;
    args.stream = stream;
    return solution->execute(args);
}
