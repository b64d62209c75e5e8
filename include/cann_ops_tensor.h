/*
 * cann_ops_tensor.h - public C API of the ops-tensor host library, B200 build.
 *
 * Part 1 is the API surface of the reference (include/cann_ops_tensor.h:43-213 of Atlas-Ascend-Fork/ops-tensor):
 * the same thirteen functions with the same parameter lists, ownership rules and status codes, so a client written
 * against the reference compiles and links unchanged (`aclrtStream` is a cudaStream_t here, see acl/acl.h).
 *
 * Part 2 adds the quantized contraction the reference's roadmap reserves names for
 * (acltensorCreateContraction, acltensorOperationDescriptorSetAttribute / GetAttribute:
 * lib/core/operation_descriptor.cpp:183-189; acltensorEstimateWorkspaceSize: lib/core/plan_preference.cpp:58;
 * acltensorContract: docs/implementation.md:68-74).  It is the host entry to the Blaze matmul path
 * (include/blaze/gemm/kernel/kernel_qbmm_mx.h, kernel_matmul_streamk.h) re-built for sm_100a.
 *
 * Conventions, as in the reference: every Create* returns a heap object through its out-parameter
 * (ALLOC_FAILED when that fails); every Destroy* accepts NULL; an operation descriptor keeps non-owning pointers to
 * its tensor descriptors and a plan keeps non-owning pointers to its operation descriptor and preference, so the
 * caller keeps those alive; errors are status codes only.
 */
#ifndef CANN_OPS_TENSOR_H
#define CANN_OPS_TENSOR_H

#include <stddef.h>

#include "cann_ops_tensor_types.h"
#include "acl/acl.h"

#if defined(_WIN32) || defined(__CYGWIN__)
#define ACLTENSOR_API __declspec(dllexport)
#else
#define ACLTENSOR_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ===================================== Part 1: reference API surface ===================================== */

/* Library handle (reference :43, :50).  Creation queries the current CUDA device. */
ACLTENSOR_API acltensorStatus_t acltensorCreate(acltensorHandle_t* handle);
ACLTENSOR_API acltensorStatus_t acltensorDestroy(acltensorHandle_t handle);

/* Tensor descriptor (reference :67-74, :81).  stridesIn == NULL means packed row-major.  Extents and strides
 * count elements (for ACLTENSOR_R_4F_E2M1, two elements share a byte). */
ACLTENSOR_API acltensorStatus_t acltensorCreateTensorDescriptor(const acltensorHandle_t handle,
                                                                acltensorTensorDescriptor_t* desc, const uint32_t rank,
                                                                const int64_t dimSizes[], const int64_t stridesIn[],
                                                                acltensorDataType_t dType, uint32_t alignReq);
ACLTENSOR_API acltensorStatus_t acltensorDestroyTensorDescriptor(acltensorTensorDescriptor_t desc);

/* D = opAC(alpha * opA(A), gamma * opC(C)) (reference :104-116, :123). */
ACLTENSOR_API acltensorStatus_t acltensorCreateElementwiseBinary(
    const acltensorHandle_t handle, acltensorOperationDescriptor_t* desc, const acltensorTensorDescriptor_t descA,
    const int32_t modeA[], acltensorOperator_t opA, const acltensorTensorDescriptor_t descC, const int32_t modeC[],
    acltensorOperator_t opC, const acltensorTensorDescriptor_t descD, const int32_t modeD[], acltensorOperator_t opAC,
    const acltensorComputeDescriptor_t descCompute);
ACLTENSOR_API acltensorStatus_t acltensorDestroyOperationDescriptor(acltensorOperationDescriptor_t desc);

/* Plan preference and plan (reference :136-139, :146, :157-162, :169). */
ACLTENSOR_API acltensorStatus_t acltensorCreatePlanPreference(const acltensorHandle_t handle,
                                                              acltensorPlanPreference_t* pref, acltensorAlgo_t algo);
ACLTENSOR_API acltensorStatus_t acltensorDestroyPlanPreference(acltensorPlanPreference_t pref);
ACLTENSOR_API acltensorStatus_t acltensorCreatePlan(const acltensorHandle_t handle, acltensorPlan_t* plan,
                                                    const acltensorOperationDescriptor_t desc,
                                                    const acltensorPlanPreference_t pref, uint64_t workspaceSizeLimit);
ACLTENSOR_API acltensorStatus_t acltensorDestroyPlan(acltensorPlan_t plan);

/* Execute an elementwise-binary plan (reference :188-196).  Asynchronous on `stream`. */
ACLTENSOR_API acltensorStatus_t acltensorElementwiseBinaryExecute(const acltensorHandle_t handle,
                                                                  const acltensorPlan_t plan, const void* alpha,
                                                                  const void* A, const void* gamma, const void* C,
                                                                  void* D, aclrtStream stream);

/* Utilities (reference :207, :213). */
ACLTENSOR_API const char* acltensorGetErrorString(const acltensorStatus_t error);
ACLTENSOR_API size_t acltensorGetVersion(void);

/* ===================================== Part 2: quantized contraction ===================================== */

/*
 * D[m,n] = act( sum_k A[m,k] * B[(g,) n,k] + bias[n] ) + C[m,n]
 *
 *   descA  rank 2, modes {m,k}, k contiguous, ACLTENSOR_R_8F_E4M3
 *   descB  rank 2 {n,k} (or {k,n} with k contiguous), or rank 3 {g,n,k} for a grouped matmul with one weight per
 *          group; ACLTENSOR_R_8F_E4M3, or ACLTENSOR_R_4F_E2M1 with MX scales
 *   descC  optional residual with the extents of D (NULL: none), ACLTENSOR_R_16BF
 *   descD  rank 2 {m,n}, n contiguous, ACLTENSOR_R_16BF
 *   opA, opB, opC must be ACLTENSOR_OP_IDENTITY; descCompute must be ACLTENSOR_COMPUTE_DESC_32F.
 * Scale modes, epilogue activation, bias, group count and scheduling hints are attributes (below).
 */
ACLTENSOR_API acltensorStatus_t acltensorCreateContraction(
    const acltensorHandle_t handle, acltensorOperationDescriptor_t* desc, const acltensorTensorDescriptor_t descA,
    const int32_t modeA[], acltensorOperator_t opA, const acltensorTensorDescriptor_t descB, const int32_t modeB[],
    acltensorOperator_t opB, const acltensorTensorDescriptor_t descC, const int32_t modeC[], acltensorOperator_t opC,
    const acltensorTensorDescriptor_t descD, const int32_t modeD[], const acltensorComputeDescriptor_t descCompute);

/* Attributes are int32 values (see acltensorOperationDescriptorAttribute_t); sizeInBytes must be 4. */
ACLTENSOR_API acltensorStatus_t acltensorOperationDescriptorSetAttribute(const acltensorHandle_t handle,
                                                                         acltensorOperationDescriptor_t desc,
                                                                         acltensorOperationDescriptorAttribute_t attr,
                                                                         const void* buf, size_t sizeInBytes);
ACLTENSOR_API acltensorStatus_t acltensorOperationDescriptorGetAttribute(const acltensorHandle_t handle,
                                                                         const acltensorOperationDescriptor_t desc,
                                                                         acltensorOperationDescriptorAttribute_t attr,
                                                                         void* buf, size_t sizeInBytes);

/* Workspace a plan for `desc` would ask for.  MIN never selects stream-K (no fix-up buffer). */
ACLTENSOR_API acltensorStatus_t acltensorEstimateWorkspaceSize(const acltensorHandle_t handle,
                                                               const acltensorOperationDescriptor_t desc,
                                                               const acltensorPlanPreference_t pref,
                                                               const acltensorWorksizePreference_t workspacePref,
                                                               uint64_t* workspaceSizeEstimate);

/* Workspace bytes the plan needs at execution (0 for elementwise plans). */
ACLTENSOR_API acltensorStatus_t acltensorPlanGetRequiredWorkspace(const acltensorPlan_t plan, uint64_t* bytes);

/*
 * Plan cache of a handle: contraction problem signature -> kernel choice (tile width, 1- or 2-CTA tiles, scheduler
 * mode).  The reference reserves these three names and leaves them unimplemented (lib/core/handle.cpp:105-108,
 * docs/implementation.md:62-64).  A plan whose descriptor leaves the choice open takes it from the cache when the
 * signature is there.  A plan created with ACLTENSOR_ALGO_DEFAULT_PATIENT (include/cann_ops_tensor_types.h:113) and
 * no cached entry times its candidates on the device during its first acltensorContract call (which therefore runs
 * the product several times and synchronises the stream), keeps the fastest and stores it in the cache.
 * The file is text: the line "acltensor-plan-cache 1", then "<signature> <tileN> <ctaPair> <splitPolicy>" per entry.
 * A missing or unreadable file gives IO_ERROR, a damaged one INVALID_VALUE and leaves the cache as it was.
 */
ACLTENSOR_API acltensorStatus_t acltensorHandleResizePlanCache(acltensorHandle_t handle, const uint32_t numEntries);
ACLTENSOR_API acltensorStatus_t acltensorHandleWritePlanCacheToFile(const acltensorHandle_t handle,
                                                                    const char filename[]);
ACLTENSOR_API acltensorStatus_t acltensorHandleReadPlanCacheFromFile(acltensorHandle_t handle, const char filename[],
                                                                     uint32_t* numCachelinesRead);
/* What the plan runs with (0 / ACLTENSOR_SPLIT_AUTO = left to the launch layer); *pendingTuning = 1 while a PATIENT
 * plan has not timed its candidates yet.  Any out-pointer may be NULL. */
ACLTENSOR_API acltensorStatus_t acltensorPlanGetKernelChoice(const acltensorPlan_t plan, int32_t* tileN,
                                                             int32_t* ctaPair, int32_t* splitPolicy,
                                                             int32_t* pendingTuning);

/* Device pointers that accompany the operands of a contraction.  Unused ones are NULL. */
typedef struct {
    const void* scaleA;    /* scales of A, layout given by SCALE_MODE_A */
    const void* scaleB;    /* scales of B, layout given by SCALE_MODE_B */
    const void* bias;      /* bf16[n], when BIAS_TYPE is set */
    const void* groupList; /* int64[groups]: rows of A per group, when GROUP_COUNT > 0 */
    void* scaleD;          /* output, when SCALE_MODE_D is set: E8M0 [m][ceil(n/64)*2] or float32 [m][ceil(n/128)] */
} acltensorContractionAux_t;

/*
 * Execute a contraction plan, asynchronously on `stream`.  alpha must be NULL or point to 1.0f; beta must be NULL,
 * 0.0f (ignore C) or 1.0f.  `workspace` is device memory, 256-byte aligned, of at least the plan's required size
 * (INSUFFICIENT_WORKSPACE otherwise).  Waits inside the kernels are bounded; one that gives up is reported by
 * acltensorGetDeviceStatus, not by this call.
 */
ACLTENSOR_API acltensorStatus_t acltensorContract(const acltensorHandle_t handle, const acltensorPlan_t plan,
                                                  const void* alpha, const void* A, const void* B, const void* beta,
                                                  const void* C, void* D, const acltensorContractionAux_t* aux,
                                                  void* workspace, uint64_t workspaceSize, aclrtStream stream);

/* Quantise fp32 device data into the operand + scale layouts a contraction consumes.  `scaleMode` selects the
 * format: MX_E8M0_VEC32 (dType E4M3 or E2M1), FP32_1X128 or FP32_128X128 (dType E4M3).  src is [rows][ldSrc]. */
ACLTENSOR_API acltensorStatus_t acltensorQuantize(const acltensorHandle_t handle, const void* src, int64_t ldSrc,
                                                  int64_t rows, int64_t cols, acltensorScaleMode_t scaleMode,
                                                  acltensorDataType_t dType, void* codes, int64_t ldCodesBytes,
                                                  void* scales, aclrtStream stream);

/* Synchronises the device and returns ACLTENSOR_STATUS_EXECUTION_FAILED if a kernel of this library abandoned a
 * wait since the last query (the code of the first such wait is stored in *deviceCode when not NULL). */
ACLTENSOR_API acltensorStatus_t acltensorGetDeviceStatus(const acltensorHandle_t handle, int32_t* deviceCode);

#ifdef __cplusplus
}
#endif
#endif /* CANN_OPS_TENSOR_H */
