/*
 * A plain C (C99) client of the drop-in boundary: includes the public headers the way a C program would, links
 * against libops_tensor_b200.so and walks the reference's call sequence for the one operator it ships (ADD:
 * src/add/tests/add_test.cpp:27-104) up to plan creation, then the contraction descriptor / attribute / plan flow, all
 * of which run on the host.  Exit code 0 = every call returned what the interface promises.
 */
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "blaze_b200.h"
#include "cann_ops_tensor.h"

#define CHECK(cond)                                                     \
    do {                                                                \
        if (!(cond)) {                                                  \
            fprintf(stderr, "line %d: %s\n", __LINE__, #cond);          \
            return 1;                                                   \
        }                                                               \
    } while (0)

int main(void) {
    acltensorHandle_t handle = NULL;
    CHECK(acltensorCreate(NULL) == ACLTENSOR_STATUS_INVALID_VALUE);
    CHECK(acltensorCreate(&handle) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorGetVersion() == ((size_t)1 << 16));
    CHECK(strlen(acltensorGetErrorString(ACLTENSOR_STATUS_NOT_SUPPORTED)) > 0);

    /* elementwise ADD: descriptors -> operation -> preference -> plan */
    const int64_t lens[1] = {1024};
    const int32_t modes[1] = {0};
    acltensorTensorDescriptor_t dA = NULL, dC = NULL, dD = NULL;
    CHECK(acltensorCreateTensorDescriptor(handle, &dA, 1, lens, NULL, ACLTENSOR_R_32F, 256) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorCreateTensorDescriptor(handle, &dC, 1, lens, NULL, ACLTENSOR_R_32F, 256) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorCreateTensorDescriptor(handle, &dD, 1, lens, NULL, ACLTENSOR_R_32F, 256) == ACLTENSOR_STATUS_SUCCESS);
    acltensorOperationDescriptor_t add = NULL;
    CHECK(acltensorCreateElementwiseBinary(handle, &add, dA, modes, ACLTENSOR_OP_IDENTITY, dC, modes,
                                           ACLTENSOR_OP_IDENTITY, dD, modes, ACLTENSOR_OP_ADD,
                                           ACLTENSOR_COMPUTE_DESC_32F) == ACLTENSOR_STATUS_SUCCESS);
    acltensorPlanPreference_t pref = NULL;
    CHECK(acltensorCreatePlanPreference(handle, &pref, ACLTENSOR_ALGO_DEFAULT) == ACLTENSOR_STATUS_SUCCESS);
    acltensorPlan_t plan = NULL;
    CHECK(acltensorCreatePlan(handle, &plan, add, pref, 0) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyPlan(plan) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyOperationDescriptor(add) == ACLTENSOR_STATUS_SUCCESS);

    /* MXFP8 contraction 256 x 512 x 1024 with bias + GELU: descriptor, attributes, workspace estimate, plan */
    const int64_t lensA[2] = {256, 1024}, lensB[2] = {512, 1024}, lensD[2] = {256, 512};
    const int32_t mA[2] = {0, 2}, mB[2] = {1, 2}, mD[2] = {0, 1};
    acltensorTensorDescriptor_t qA = NULL, qB = NULL, qD = NULL;
    CHECK(acltensorCreateTensorDescriptor(handle, &qA, 2, lensA, NULL, ACLTENSOR_R_8F_E4M3, 256) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorCreateTensorDescriptor(handle, &qB, 2, lensB, NULL, ACLTENSOR_R_8F_E4M3, 256) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorCreateTensorDescriptor(handle, &qD, 2, lensD, NULL, ACLTENSOR_R_16BF, 256) == ACLTENSOR_STATUS_SUCCESS);
    acltensorOperationDescriptor_t mm = NULL;
    CHECK(acltensorCreateContraction(handle, &mm, qA, mA, ACLTENSOR_OP_IDENTITY, qB, mB, ACLTENSOR_OP_IDENTITY, NULL,
                                     NULL, ACLTENSOR_OP_IDENTITY, qD, mD,
                                     ACLTENSOR_COMPUTE_DESC_32F) == ACLTENSOR_STATUS_SUCCESS);
    int32_t v = ACLTENSOR_SCALE_MX_E8M0_VEC32;
    CHECK(acltensorOperationDescriptorSetAttribute(handle, mm, ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_A, &v,
                                                   sizeof(v)) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorOperationDescriptorSetAttribute(handle, mm, ACLTENSOR_OPERATION_DESCRIPTOR_SCALE_MODE_B, &v,
                                                   sizeof(v)) == ACLTENSOR_STATUS_SUCCESS);
    v = ACLTENSOR_OP_GELU;
    CHECK(acltensorOperationDescriptorSetAttribute(handle, mm, ACLTENSOR_OPERATION_DESCRIPTOR_EPILOGUE_ACT, &v,
                                                   sizeof(v)) == ACLTENSOR_STATUS_SUCCESS);
    v = ACLTENSOR_OP_SQRT;
    CHECK(acltensorOperationDescriptorSetAttribute(handle, mm, ACLTENSOR_OPERATION_DESCRIPTOR_EPILOGUE_ACT, &v,
                                                   sizeof(v)) == ACLTENSOR_STATUS_NOT_SUPPORTED);
    v = 0;
    CHECK(acltensorOperationDescriptorGetAttribute(handle, mm, ACLTENSOR_OPERATION_DESCRIPTOR_EPILOGUE_ACT, &v,
                                                   sizeof(v)) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(v == ACLTENSOR_OP_GELU);
    uint64_t estimate = 0, need = 0;
    CHECK(acltensorEstimateWorkspaceSize(handle, mm, pref, ACLTENSOR_WORKSPACE_DEFAULT, &estimate) ==
          ACLTENSOR_STATUS_SUCCESS);
    CHECK(estimate > 0);
    CHECK(acltensorCreatePlan(handle, &plan, mm, pref, 0) == ACLTENSOR_STATUS_INSUFFICIENT_WORKSPACE);
    CHECK(acltensorCreatePlan(handle, &plan, mm, pref, estimate) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorPlanGetRequiredWorkspace(plan, &need) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(need > 0 && need <= estimate);
    /* executing needs device pointers; a missing one is reported, not dereferenced */
    acltensorContractionAux_t aux;
    memset(&aux, 0, sizeof(aux));
    CHECK(acltensorContract(handle, plan, NULL, NULL, NULL, NULL, NULL, NULL, &aux, NULL, 0, NULL) ==
          ACLTENSOR_STATUS_INVALID_VALUE);

    /* the kernel ABI is reachable from C as well: a workspace query runs on the host */
    blazeMxGemmArgs args;
    memset(&args, 0, sizeof(args));
    args.struct_size = sizeof(args);
    args.M = 256;
    args.N = 512;
    args.K = 1024;
    size_t bytes = 0;
    CHECK(blazeMxGemmWorkspaceSize(&args, &bytes) == ACLTENSOR_STATUS_SUCCESS && bytes > 0);
    args.K = 1000;
    CHECK(blazeMxGemmWorkspaceSize(&args, &bytes) == ACLTENSOR_STATUS_NOT_SUPPORTED);

    CHECK(acltensorDestroyPlan(plan) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyPlanPreference(pref) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyOperationDescriptor(mm) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyTensorDescriptor(dA) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyTensorDescriptor(dC) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyTensorDescriptor(dD) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyTensorDescriptor(qA) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyTensorDescriptor(qB) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyTensorDescriptor(qD) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroyTensorDescriptor(NULL) == ACLTENSOR_STATUS_SUCCESS);
    CHECK(acltensorDestroy(handle) == ACLTENSOR_STATUS_SUCCESS);
    printf("c client ok: workspace estimate %llu bytes\n", (unsigned long long)estimate);
    return 0;
}
